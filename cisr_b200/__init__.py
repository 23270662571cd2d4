"""Import name of the engine.

The sources live in the folder ``cuda-inference-serving-runtime_b200/`` beside this
one; a hyphen cannot appear in an import statement, so this package points its
search path there and runs that folder's ``__init__.py`` as its own.
"""
from pathlib import Path as _Path

_SRC = _Path(__file__).resolve().parent.parent / "cuda-inference-serving-runtime_b200"
__path__ = [str(_SRC)]
exec(compile((_SRC / "__init__.py").read_text(), str(_SRC / "__init__.py"), "exec"))
