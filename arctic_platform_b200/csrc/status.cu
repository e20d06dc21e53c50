// Kernel status word, tensor-map encoding through the driver entry point and
// small exported utilities (status read/clear, L2 flush helper).
#include "host_utils.cuh"
#include <stdlib.h>

namespace apb {

__device__ int g_status_word[4];

int* status_device_ptr() {
  // One address per device; looked up on first use with that device current.
  static int* ptrs[64] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (!ptrs[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    ptrs[dev] = static_cast<int*>(p);
  }
  return ptrs[dev];
}

static int g_chained_launch = 0;
bool chained_launch_on() { return g_chained_launch != 0; }

int sm_count() {
  static int n[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (!n[dev]) cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
  return n[dev] > 0 ? n[dev] : 148;
}

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

int make_tmap_2d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t ld,
                 uint32_t box_cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return -1;
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                             : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

int make_tmap_nd(CUtensorMap* map, const void* base, int elem_bytes, int rank, const uint64_t* dims,
                 const uint64_t* strides_bytes, const uint32_t* box) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn || rank < 1 || rank > 5) return -1;
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                             : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t d[5];
  cuuint64_t st[4];
  cuuint32_t bx[5];
  cuuint32_t es[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i > 0) st[i - 1] = strides_bytes[i - 1];
  }
  CUresult r = fn(map, dt, rank, const_cast<void*>(base), d, st, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

__global__ void fill_u32_kernel(uint32_t* p, size_t n, uint32_t v) {
  size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (; i < n; i += stride) p[i] = v;
}

}  // namespace apb

extern "C" {

// Reads the status word of the current device (0 = no kernel reported an error).
int apb_status_read() {
  int* p = apb::status_device_ptr();
  if (!p) return -1;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  return v;
}

// The whole record: {code, expected epoch, peer, epoch seen} -- the last three are filled by a timed-out wait on a
// peer's flag and are zero otherwise.
int apb_status_read4(int* out4) {
  int* p = apb::status_device_ptr();
  if (!p || !out4) return -1;
  return cudaMemcpy(out4, p, 4 * sizeof(int), cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : -2;
}

int apb_status_clear() {
  int* p = apb::status_device_ptr();
  if (!p) return -1;
  return static_cast<int>(cudaMemset(p, 0, 4 * sizeof(int)));
}

// Overwrites `bytes` of `buf` (used by benchmarks to flush the L2 between timed iterations).
int apb_fill_u32(void* buf, size_t bytes, uint32_t value, cudaStream_t stream) {
  apb::fill_u32_kernel<<<1184, 256, 0, stream>>>(static_cast<uint32_t*>(buf), bytes / 4, value);
  return static_cast<int>(cudaGetLastError());
}

// Makes `dev` the current device of the calling thread for this library's CUDA runtime instance.
// The Python wrappers call it before every launch: autograd worker threads and freshly started
// threads have no device bound in this (statically linked) runtime, and tensor-map encoding needs
// a current context.
int apb_bind_device(int dev) {
  static thread_local int bound = -1;
  if (bound == dev) return 0;
  cudaError_t e = cudaSetDevice(dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaFree(0);
  if (e != cudaSuccess) return static_cast<int>(e);
  bound = dev;
  return 0;
}

// Switches chained launches on or off for this process and returns the previous setting.  While on, the kernels
// of this library that support it are launched with the programmatic-serialization attribute and the GEMM
// prefetches its B operand before waiting for the previous kernel: only valid while B (the weights) is not
// written by any kernel of the chain, i.e. during a decode step.  APB_PDL=0 in the environment keeps it off.
int apb_set_chained_launch(int on) {
  static int allowed = -1;
  if (allowed < 0) {
    const char* e = getenv("APB_PDL");
    allowed = (e && e[0] == '0') ? 0 : 1;
  }
  const int prev = apb::g_chained_launch;
  apb::g_chained_launch = (on && allowed) ? 1 : 0;
  return prev;
}

int apb_version() { return 2; }
}
