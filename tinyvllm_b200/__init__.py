"""Import name of the package whose sources live in the folder ``tiny-vllm_b200``.

A folder name with a hyphen cannot be imported, so this module points the
package search path at that folder and runs its ``__init__``; every submodule
(``tinyvllm_b200.engine`` and so on) then resolves there.
"""

from pathlib import Path as _Path

_SOURCE = _Path(__file__).resolve().parent.parent / "tiny-vllm_b200"
__path__ = [str(_SOURCE)]
__file__ = str(_SOURCE / "__init__.py")
exec(compile((_SOURCE / "__init__.py").read_text(encoding="utf-8"), __file__, "exec"))
