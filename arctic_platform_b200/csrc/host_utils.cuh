// Host-side helpers shared by the .cu files: the kernel status word, the
// driver entry point for tensor-map encoding and a 2-D bf16/fp8 tensor-map
// builder with 128-byte swizzle.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace apb {

// Device status word shared by every kernel of the library.  Defined once in
// status.cu; kernels receive its device address as a parameter.
int* status_device_ptr();

// Multiprocessor count of the current device (cached per device; 148 on a B200).
int sm_count();

// Chained-launch mode (see apb_set_chained_launch in status.cu): while it is on, kernels go out with the
// programmatic-serialization attribute, so that each may start (set-up, weight prefetch) before the previous
// one has finished; every such kernel calls pdl_wait() before it touches data of its predecessor.
bool chained_launch_on();

// Launch helper used instead of <<<>>> by the kernels that take part in chained launches.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = chained_launch_on() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn();

// Row-major 2-D tensor [rows, cols] with `ld` elements between rows; box is
// box_cols x box_rows elements, 128-byte swizzle (box_cols * elem_bytes must
// be 128).  Returns 0 on success.
int make_tmap_2d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t ld,
                 uint32_t box_cols, uint32_t box_rows);

// General tiled tensor map (rank <= 5), 128-byte swizzle.  dims/box innermost first; strides in BYTES for
// dimensions 1..rank-1 (dimension 0 is contiguous).
int make_tmap_nd(CUtensorMap* map, const void* base, int elem_bytes, int rank, const uint64_t* dims,
                 const uint64_t* strides_bytes, const uint32_t* box);

}  // namespace apb
