"""ABI markers shared by the Python control plane and the native extension."""

CORE_ABI_VERSION = 1
# Reference parity: ccdl_comm/abi.py:3 exposes CCDL_CORE_ABI = 1.
CCDL_CORE_ABI = CORE_ABI_VERSION
NATIVE_WORK_ABI_VERSION = 1
