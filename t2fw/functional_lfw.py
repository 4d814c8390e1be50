"""Import-path alias: `from t2fw.functional_lfw import LFWFunction` keeps working."""
from t2fw_b200.functional_lfw import LFWFunction  # noqa: F401
