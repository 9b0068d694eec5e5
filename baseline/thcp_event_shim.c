/* torch 2.11 no longer exports the data symbol `THCPEventClass` from
 * libtorch_python.so, but torch/csrc/cuda/Event.h still declares it and the
 * reference's extension (csrc/executor/compressed_work.cpp) references it, so
 * its shared object cannot be loaded as built.  This one-variable library
 * supplies the symbol; reference_env.py loads it with RTLD_GLOBAL and points it
 * at torch._C._CudaEventBase, which is the object the symbol named in older
 * torch releases.  The reference itself is not modified. */
#include <Python.h>

PyObject* THCPEventClass = NULL;
