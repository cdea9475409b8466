/* ref_py.c — the reference's Python-facing C shim (py/csrc/libthvm.m: the `py_*` functions its ctypes layer
 * py/tinyhvm/_ffi.py binds) compiled from the source where it lies in the reference checkout, together with the CUDA
 * backend hub.  TEST INFRASTRUCTURE ONLY; nothing of the reference is copied.
 *
 * The shim's py_init calls thvm_init, which ignores its device argument off Apple (src/ctx/init.c:36-38).  The whole
 * translation unit is compiled with thvm_init renamed, and py_init_device below is what py_init becomes once
 * thvm_init has the "cuda" branch of the hub: py_init_device("cuda") brings up libthvm_cuda.so behind
 * the same surface a Python user of the reference sees, py_init_device("cpu") keeps the reference's CPU backend. */
#define thvm_init thvm_init_base
#include "py/csrc/libthvm.m"
#undef thvm_init
#include "../tinyhvm_b200/backend_cuda/_.c"

__attribute__((visibility("default")))
TinyHVM *py_init_device(const char *device) { return thvm_init_device(thvm_init_base, device); }
