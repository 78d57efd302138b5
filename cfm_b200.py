"""Import alias for the package directory `calibration-free-moe_b200/`.

The directory name contains a hyphen, which Python's import statement cannot
spell.  Importing this module registers that directory as the package
`cfm_b200`, so `import cfm_b200` and `from cfm_b200.reader import ...` work
from the repository root.
"""

import importlib.util
import pathlib
import sys

_directory = pathlib.Path(__file__).resolve().parent / "calibration-free-moe_b200"
_spec = importlib.util.spec_from_file_location(
    __name__,
    _directory / "__init__.py",
    submodule_search_locations=[str(_directory)],
)
_package = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _package
_spec.loader.exec_module(_package)
