"""Test-only distributed op registered through HYPER_PARALLEL_OPS_YAML_DIR / _PYTHON_PATH:
``stack_rows(a, b)`` stacks two equally laid-out tensors along a new leading (unsharded) dim."""
from hyper_parallel_b200 import DistributedOp


class StackDistributedOp(DistributedOp):
    def infer_layout(self, layouts, extra_args):
        a, b = layouts[0], layouts[1]
        if tuple(a.alias_tensor_map) != tuple(b.alias_tensor_map):
            raise ValueError("stack_rows needs identically sharded inputs")
        return a("None", *a.alias_tensor_map)
