"""`pip install .` packages the Python sources and the kernel sources.

Native code is built in-tree, not by pip: `python -m lowbit_comm_b200.ops.build` (nvcc -gencode
arch=compute_100a,code=sm_100a plus g++) writes `_lbc_cuda.so` and `_lbc_host.so` next to `ops/`, and an
install made afterwards carries them.  Set LBC_BUILD_NATIVE=1 to run that build as part of `pip install`
(needs torch and the CUDA toolkit at build time; `LBC_BUILD_NATIVE=host` builds only the g++ host codec).

Role parity: the reference's extension spec and split distributions
(ccdl_comm/build/extension.py:33-76, build/distributions.py); one distribution here, one optional switch.
"""

import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py


class BuildWithNative(build_py):
    def run(self):
        mode = os.environ.get("LBC_BUILD_NATIVE", "").lower()
        if mode in ("1", "true", "cuda", "host"):
            sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
            from lowbit_comm_b200.ops import build as native

            native.build_host_library()
            if mode != "host":
                native.build_extension()
        super().run()


setup(cmdclass={"build_py": BuildWithNative})
