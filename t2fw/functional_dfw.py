"""Import-path alias: `from t2fw.functional_dfw import DFWFunction` keeps working."""
from t2fw_b200.functional_dfw import DFWFunction  # noqa: F401
