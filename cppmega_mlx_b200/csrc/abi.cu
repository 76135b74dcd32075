// ABI handshake between the Python package and the kernel library. The loader refuses a library
// whose version differs from the one the Python sources were written against. Same purpose as the
// reference's native-bridge probe (cppmega_mlx/nn/_tilelang/native_bridge/tilelang_mlx_tvm_ffi_bridge.cpp:32-70).
#include <cuda_runtime.h>

extern "C" int cmb_abi_version() { return 3; }

extern "C" int cmb_device_sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
  return n;
}
