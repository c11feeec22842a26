"""`import mamtorch` for code written against SSIGPRO/mamtorch: the name resolves to `mamtorch_b200`.

After this import `mamtorch`, `mamtorch.kernel.v1 ... v4`, `mamtorch.nn`, `mamtorch.nn.v4`,
`mamtorch.sparse.kernel.v1` and `mamtorch.MAMDense` are the modules and classes of `mamtorch_b200`
(the same objects, not copies), matching the import surface of the reference's `mamtorch/__init__.py:1-7`.
A process can hold only one implementation of the `torch.ops.mamtorch_kernel_v*` operators: if the
reference's own extension modules are already loaded, loading this package fails in the operator
registration instead of silently mixing the two.
"""
import sys

import mamtorch_b200 as _impl

for _name, _mod in list(sys.modules.items()):
    if _name.startswith("mamtorch_b200."):
        sys.modules[__name__ + _name[len("mamtorch_b200"):]] = _mod
sys.modules[__name__] = _impl
