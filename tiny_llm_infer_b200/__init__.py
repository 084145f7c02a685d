"""Importable name of the package whose sources live in ``tiny-llm-infer_b200/``.

A folder name with a hyphen cannot appear in an ``import`` statement, so this
module points its ``__path__`` at that folder and runs the folder's own
``__init__.py``.  ``import tiny_llm_infer_b200.engine`` therefore loads
``tiny-llm-infer_b200/engine/__init__.py``.
"""
from pathlib import Path as _Path

_SRC = _Path(__file__).resolve().parent.parent / "tiny-llm-infer_b200"
if not (_SRC / "__init__.py").is_file():
    raise ImportError(f"package sources not found at {_SRC}")
__path__ = [str(_SRC)]
__file__ = str(_SRC / "__init__.py")
exec(compile((_SRC / "__init__.py").read_text(), __file__, "exec"))
