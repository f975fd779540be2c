"""The compiler entry points of the reference, by name (newt/compiler/__init__.py):
`newt_b200.compiler.codegen.compile_fn` and `newt_b200.compiler.types`.  The work is done by
newt_b200/frontend (trace -> launch plan, generated CUDA where no tuned kernel applies)."""

from .. import types  # noqa: F401
from . import codegen  # noqa: F401
