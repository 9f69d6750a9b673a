// Host-side helpers shared by the kernels: error codes, driver entry point for tensor-map
// encoding (resolved at run time so the library loads on machines without a driver), and
// tensor-map builders for 128-byte-swizzled tiles.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <utility>

namespace tp {

enum ErrorCode : int {
  kOk = 0,
  kErrBadArgument = -1,
  kErrDriver = -2,
  kErrLaunch = -3,
  kErrTooLarge = -4,
  // device-side wait time-outs (written to the caller's error word)
  kErrWaitProducer = 101,
  kErrWaitMma = 102,
  kErrWaitEpilogue = 103,
  kErrWaitTmemEmpty = 104,
  kErrWaitPeer = 105,
  kErrWaitAttn = 106,
  // checked build only: an index check inside a kernel failed (the access was skipped)
  kErrCheckTile = 121,      // GEMM tile outside the output grid
  kErrCheckStaging = 122,   // slot of a peer staging / flag array beyond its capacity
  kErrCheckPeer = 123,      // rank index outside the group
  kErrCheckAttn = 124,      // attention row or key block outside the buffers
  kErrCheckNorm = 125,      // LayerNorm / element-wise row, column or slot outside the buffers
  kErrCheckSelfTest = 129,  // raised on purpose by tp_checked_selftest
};

// Checked build (-DTP_CHECKED, loaded with TERAPIPE_CHECKED=1): index checks compiled into the
// kernels next to the accesses that no tensor map bounds (raw pointers into peer staging, flag
// arrays, partial-sum slots).  A failed check writes its code into the launch's status word
// (the first failure wins) and the guarded access is skipped; nothing traps, so the context
// stays usable and the host reads the code like a wait time-out.  In the regular build
// TP_CHECK(...) is the constant `true` and its condition is not evaluated.
#ifdef TP_CHECKED
#ifdef __CUDACC__
__device__ __forceinline__ bool check_record(bool ok, int* err, int code) {
  if (!ok && err != nullptr) atomicCAS(err, 0, code);
  return ok;
}
#endif
#define TP_CHECK(cond, err, code) (::tp::check_record((cond), (err), (code)))
#else
#define TP_CHECK(cond, err, code) (true)
#endif

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 16-bit elements, 128B swizzle.  dims/strides innermost first; strides[i] is the byte stride
// of dimension i+1.  Returns false on failure.
inline bool make_tmap_16b(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                          const uint64_t* strides_bytes, const uint32_t* box, bool bf16) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(out, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                  rank, const_cast<void*>(base), reinterpret_cast<const cuuint64_t*>(dims),
                  reinterpret_cast<const cuuint64_t*>(strides_bytes), box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "terapipe_b200: cuTensorMapEncodeTiled failed (%d) rank=%d dims=%llu,%llu box=%u,%u stride=%llu base=%p\n",
            (int)r, rank, (unsigned long long)dims[0], (unsigned long long)dims[1], box[0], box[1],
            (unsigned long long)strides_bytes[0], base);
    return false;
  }
  return true;
}

inline bool make_tmap_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                         uint64_t ld_elems, uint32_t box_inner, uint32_t box_outer, bool bf16) {
  uint64_t dims[2] = {inner, outer};
  uint64_t strides[1] = {ld_elems * 2};
  uint32_t box[2] = {box_inner, box_outer};
  return make_tmap_16b(out, base, 2, dims, strides, box, bf16);
}

// Tensor map of a row-major [rows][cols] output matrix for the epilogue's staged stores: boxes
// of 32 x 32 elements whose shared-memory rows are 64 bytes (16-bit elements, 64-byte swizzle)
// or 128 bytes (fp32, 128-byte swizzle).
inline bool make_tmap_out(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows,
                          uint64_t ld_elems, bool f32, bool bf16) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {ld_elems * (f32 ? 4u : 2u)};
  const cuuint32_t box[2] = {32, 32};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                     : (bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  f32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "terapipe_b200: cuTensorMapEncodeTiled (output map) failed (%d) dims=%llu,%llu ld=%llu base=%p\n",
            (int)r, (unsigned long long)cols, (unsigned long long)rows, (unsigned long long)ld_elems, base);
    return false;
  }
  return true;
}

// Launch with programmatic stream serialization (see pdl_wait in ptx.cuh).  The kernel must call
// pdl_wait() in every thread before its first access to global data.  The attribute is off
// unless tp_set_pdl(1) was called or the environment variable TERAPIPE_PDL=1 is set at first use
// (it measured no gain on a step that runs at the power cap: time saved in gaps came back as a
// lower clock).
inline int& pdl_enabled() {
  static int enabled = -1;
  if (enabled < 0) {
    const char* e = getenv("TERAPIPE_PDL");
    enabled = (e && e[0] == '1') ? 1 : 0;
  }
  return enabled;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, int cluster_x, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

inline int num_sms() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace tp
