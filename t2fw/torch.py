"""Import-path alias: `from t2fw.torch import t2fw_torch, t2dfw_torch, ...` keeps working."""
from t2fw_b200.torch_loops import (t2dfw_torch, t2dfw_torch_bw, t2dfw_torch_bw_simple,  # noqa: F401
                                   t2fw_torch)
