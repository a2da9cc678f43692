"""Import alias for the package directory ``blackwell-moe-kernel-scheduler_b200``.

The directory name is not a valid Python identifier, so this module loads it
under the name ``bmoe_b200`` (sub-modules: ``bmoe_b200.engine`` and so on).
"""

import importlib.util
import sys
from pathlib import Path

_PKG_DIR = Path(__file__).resolve().parent / "blackwell-moe-kernel-scheduler_b200"

_spec = importlib.util.spec_from_file_location(
    "bmoe_b200", _PKG_DIR / "__init__.py", submodule_search_locations=[str(_PKG_DIR)]
)
_module = importlib.util.module_from_spec(_spec)
sys.modules["bmoe_b200"] = _module
_spec.loader.exec_module(_module)

if __name__ == "__main__":  # python bmoe_b200.py --kernel v2_dynamic --csv ...
    from bmoe_b200.cli import main

    main()
