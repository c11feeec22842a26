"""Operator wrappers, one sub-package per kernel generation of the reference
(`mamtorch/kernel/__init__.py`).  The reference builds and imports v1 and v4 only; v2 and v3 are
served here as well because its own test script calls them (`test/test.py:38-128`)."""
from . import v1
from . import v2
from . import v3
from . import v4
