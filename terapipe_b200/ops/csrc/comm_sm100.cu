// Peer-mapped device buffers through CUDA IPC (one process per GPU, same node).
// A buffer is a plain cudaMalloc allocation, zero-filled; its IPC handle is exchanged by the
// caller (e.g. through torch.distributed) and opened in the peers, which also turns on peer
// access over NVLink.  Kernels then read and write it with ordinary loads and stores.
#include <string.h>

#include "common.cuh"

using namespace tp;

extern "C" void* tp_symm_alloc(long long bytes) {
  void* p = nullptr;
  if (cudaMalloc(&p, static_cast<size_t>(bytes)) != cudaSuccess) return nullptr;
  if (cudaMemset(p, 0, static_cast<size_t>(bytes)) != cudaSuccess) {
    cudaFree(p);
    return nullptr;
  }
  cudaDeviceSynchronize();
  return p;
}

extern "C" int tp_symm_free(void* p) { return cudaFree(p) == cudaSuccess ? kOk : kErrDriver; }

// handle: 64 bytes
extern "C" int tp_ipc_export(void* p, unsigned char* handle) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) return kErrDriver;
  static_assert(sizeof(h) == 64, "unexpected IPC handle size");
  memcpy(handle, &h, sizeof(h));
  return kOk;
}

extern "C" void* tp_ipc_import(const unsigned char* handle) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return p;
}

extern "C" int tp_ipc_close(void* p) {
  return cudaIpcCloseMemHandle(p) == cudaSuccess ? kOk : kErrDriver;
}

// ---------------------------------------------------------------------------------------------
// Data-parallel gradient reduction fused with the optimizer (sharded update).
//
// Every data-parallel rank holds the same parameters and a full fp32 gradient buffer.  Rank r
// owns the r-th contiguous chunk of the flat parameter space.  One kernel per rank:
//   1. start handshake: tell every peer "my gradients are final" and wait for theirs;
//   2. for the owned chunk: load the chunk of EVERY rank's gradient buffer over NVLink
//      (plain peer loads), sum in fp32, scale by 1/(loss scale * replicas);
//   3. Adam on the owned chunk of the fp32 master / moment buffers (local);
//   4. store the updated 16-bit parameters into EVERY rank's model buffer (peer stores);
//   5. end handshake: the last CTA tells every peer "done" and waits for theirs, so that when the
//      kernel ends all parameters have arrived here and nobody still reads these gradients.
// Compared with all-reduce + replicated Adam this moves 4 B/param (gradients in) + 2 B/param
// (parameters out) per peer instead of 8 B/param, and updates 1/dp of the optimizer state.
// Gradients are never cleared: the producers overwrite them every iteration.
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include "ptx.cuh"

namespace tp {

constexpr int kMaxDp = 8;

struct DpParams {
  int dp, rank;
  int epoch;                  // call index; the kernel adds *epoch_base
  const int* epoch_base;
  const float* grad[kMaxDp];  // every rank's gradient buffer
  void* model[kMaxDp];        // every rank's 16-bit parameter buffer
  int* flags[kMaxDp];         // every rank's flag block: [0..dp) start flags, [dp..2dp) done flags, [2dp] counter
  float* master;
  float* m;
  float* v;
  long long begin, end;       // owned element range (multiples of 4)
  const float* adam_state;    // step, 1-beta1^t, 1-beta2^t
  float lr, beta1, beta2, eps, weight_decay, grad_scale;
  int* err;
};

__device__ __forceinline__ void st_release_sys_i(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys_i(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool spin_until(const int* p, int target, int* err, int code) {
  unsigned long long t0 = 0;
  unsigned spins = 0;
  while (ld_acquire_sys_i(p) < target) {
    if ((++spins & 0x3F) == 0) {
      if (err && *reinterpret_cast<volatile int*>(err) != 0) return false;  // already out of step
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > g_wait_limit_ns) {
        if (err) atomicCAS(err, 0, code);
        return false;
      }
    }
  }
  return true;
}

template <typename T>
__global__ void __launch_bounds__(256) dp_reduce_adam_kernel(const DpParams p) {
  __shared__ int s_ok;
  const int epoch = p.epoch + (p.epoch_base ? *p.epoch_base : 0);
  int* my_flags = p.flags[p.rank];
  if (threadIdx.x == 0) {
    if (blockIdx.x == 0)
      for (int r = 0; r < p.dp; ++r) st_release_sys_i(p.flags[r] + p.rank, epoch);
    // checked build: group size within the pointer tables, owned range well formed
    bool ok = TP_CHECK(p.dp >= 1 && p.dp <= kMaxDp && p.rank >= 0 && p.rank < p.dp, p.err, kErrCheckPeer) &&
              TP_CHECK(p.begin >= 0 && p.begin <= p.end && ((p.begin | p.end) & 3) == 0, p.err, kErrCheckNorm);
    for (int r = 0; r < p.dp && ok; ++r) ok = spin_until(my_flags + r, epoch, p.err, kErrWaitPeer);
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (s_ok) {
    const float bc1 = p.adam_state[1], bc2 = p.adam_state[2];
    const float inv_bc2_sqrt = rsqrtf(bc2);
    const float step = p.lr / bc1;
    const long long n4 = (p.end - p.begin) / 4;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      const long long e = p.begin + i * 4;
      float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
      for (int r = 0; r < p.dp; ++r) {
        const float4 t = __ldcg(reinterpret_cast<const float4*>(p.grad[r] + e));
        g.x += t.x; g.y += t.y; g.z += t.z; g.w += t.w;
      }
      float4 w4 = *reinterpret_cast<float4*>(p.master + e);
      float4 m4 = *reinterpret_cast<float4*>(p.m + e);
      float4 v4 = *reinterpret_cast<float4*>(p.v + e);
      float* gg = reinterpret_cast<float*>(&g);
      float* ww = reinterpret_cast<float*>(&w4);
      float* mm = reinterpret_cast<float*>(&m4);
      float* vv = reinterpret_cast<float*>(&v4);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float gj = gg[j] * p.grad_scale;
        mm[j] = p.beta1 * mm[j] + (1.0f - p.beta1) * gj;
        vv[j] = p.beta2 * vv[j] + (1.0f - p.beta2) * gj * gj;
        const float denom = sqrtf(vv[j]) * inv_bc2_sqrt + p.eps;
        ww[j] = ww[j] - step * (mm[j] / denom) - p.lr * p.weight_decay * ww[j];
      }
      *reinterpret_cast<float4*>(p.master + e) = w4;
      *reinterpret_cast<float4*>(p.m + e) = m4;
      *reinterpret_cast<float4*>(p.v + e) = v4;
      uint2 o;
      o.x = Elem<T>::pack2(ww[0], ww[1]);
      o.y = Elem<T>::pack2(ww[2], ww[3]);
      for (int r = 0; r < p.dp; ++r) *reinterpret_cast<uint2*>(static_cast<T*>(p.model[r]) + e) = o;
    }
  }
  // end handshake by the last CTA of this rank
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* counter = my_flags + 2 * kMaxDp;
    const int done = atomicAdd(counter, 1);
    if (done == static_cast<int>(gridDim.x) - 1) {
      *counter = 0;
      __threadfence_system();
      for (int r = 0; r < p.dp; ++r) st_release_sys_i(p.flags[r] + kMaxDp + p.rank, epoch);
      for (int r = 0; r < p.dp; ++r)
        if (!spin_until(my_flags + kMaxDp + r, epoch, p.err, kErrWaitPeer)) break;
    }
  }
}

}  // namespace tp

// grad_ptrs / model_ptrs / flag_ptrs: one address per data-parallel rank (peer mapped).  The flag
// block of a rank holds 2 * 8 + 1 ints, zero before the first call.  [begin, end) is the element
// range this rank owns; all ranks must call with the same epoch = `epoch` + *`epoch_base`,
// growing from call to call.
extern "C" int tp_dp_reduce_adam(int dtype, int dp, int rank, int epoch, const int* epoch_base,
                                 void* const* grad_ptrs, void* const* model_ptrs,
                                 void* const* flag_ptrs, float* master, float* m, float* v,
                                 long long begin, long long end, const float* adam_state, float lr,
                                 float beta1, float beta2, float eps, float weight_decay,
                                 float grad_scale, int* err, void* stream) {
  if (dp < 2 || dp > kMaxDp || rank < 0 || rank >= dp || begin % 4 || end % 4 || end < begin)
    return kErrBadArgument;
  DpParams p;
  p.dp = dp; p.rank = rank; p.epoch = epoch; p.epoch_base = epoch_base;
  for (int i = 0; i < kMaxDp; ++i) {
    p.grad[i] = i < dp ? static_cast<const float*>(grad_ptrs[i]) : nullptr;
    p.model[i] = i < dp ? model_ptrs[i] : nullptr;
    p.flags[i] = i < dp ? static_cast<int*>(flag_ptrs[i]) : nullptr;
  }
  p.master = master; p.m = m; p.v = v; p.begin = begin; p.end = end; p.adam_state = adam_state;
  p.lr = lr; p.beta1 = beta1; p.beta2 = beta2; p.eps = eps; p.weight_decay = weight_decay;
  p.grad_scale = grad_scale; p.err = err;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = 2 * num_sms();
  if (dtype == 1) dp_reduce_adam_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(p);
  else dp_reduce_adam_kernel<__half><<<grid, 256, 0, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

// ---------------------------------------------------------------------------------------------
// Link probe: how fast can SM-issued stores fill a (peer-mapped) buffer?  Used to choose the
// store pattern of the fused compute + collective kernels.
//   mode 0: every thread stores 16 bytes, a warp covers 512 contiguous bytes per instruction
//   mode 1: as 0, and each CTA runs a system-scope fence after every 32 KB (what publishing a
//           tile costs)
//   mode 2: one thread per CTA issues 16 KB bulk copies shared -> global (cp.async.bulk)
namespace tp {

__global__ void __launch_bounds__(256, 1)
link_probe_kernel(uint4* dst, long long n_vec, int mode) {
  extern __shared__ __align__(128) uint8_t probe_smem[];
  const long long per_cta = n_vec / gridDim.x;
  uint4* d = dst + static_cast<long long>(blockIdx.x) * per_cta;
  if (mode <= 1) {
    const uint4 v = make_uint4(threadIdx.x, blockIdx.x, 1u, 2u);
    long long it = 0;
    for (long long i = threadIdx.x; i < per_cta; i += blockDim.x, ++it) {
      d[i] = v;
      if (mode == 1 && (it & 7) == 7) {
        __syncthreads();
        if (threadIdx.x == 0) __threadfence_system();
      }
    }
  } else {
    constexpr int kChunk = 16384;
    for (int i = threadIdx.x; i < kChunk / 16; i += blockDim.x)
      reinterpret_cast<uint4*>(probe_smem)[i] = make_uint4(i, blockIdx.x, 1u, 2u);
    fence_proxy_async();
    __syncthreads();
    if (threadIdx.x == 0) {
      const long long n_chunks = per_cta * 16 / kChunk;
      for (long long c = 0; c < n_chunks; ++c) {
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(
                         reinterpret_cast<uint64_t>(reinterpret_cast<uint8_t*>(d) + c * kChunk)),
                     "r"(smem_u32(probe_smem)), "r"(kChunk)
                     : "memory");
        bulk_commit();
        bulk_wait_read<8>();  // bounded number of copies in flight
      }
      bulk_wait<0>();
    }
  }
}

}  // namespace tp

// Fills `bytes` (a multiple of 148 * 16 KB is best) at `dst` with the chosen store pattern.
extern "C" int tp_link_probe(void* dst, long long bytes, int mode, void* stream) {
  using namespace tp;
  if (!dst || bytes <= 0 || mode < 0 || mode > 2) return kErrBadArgument;
  const int grid = num_sms();
  const long long n_vec = bytes / 16 / grid * grid;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  link_probe_kernel<<<grid, 256, 16384, s>>>(static_cast<uint4*>(dst), n_vec, mode);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

// ---------------------------------------------------------------------------------------------
// Small collectives of the sequence-parallel tensor-parallel path (all over peer-mapped memory,
// plain loads / stores and system-scope flags, every wait bounded).
namespace tp {

struct PeerPtrs {
  void* ptr[kMaxDp];
  int* flags[kMaxDp];
  int n, rank, epoch;
  const int* epoch_base;
  int* counter;
  int* err;
};

// Copy `n_vec` 16-byte vectors from `src` (local) to the same offset of every other rank's
// buffer, then raise flags[r][rank] = epoch at every other rank r (last CTA).
__global__ void __launch_bounds__(256) ag_push_kernel(const uint4* __restrict__ src, long long n_vec,
                                                      const PeerPtrs pp) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n_vec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 v = __ldcg(src + i);
    for (int r = 0; r < pp.n; ++r)
      if (r != pp.rank) static_cast<uint4*>(pp.ptr[r])[i] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(reinterpret_cast<unsigned*>(pp.counter), 1u) == gridDim.x - 1) {
      *pp.counter = 0;
      const int epoch = pp.epoch + (pp.epoch_base ? *pp.epoch_base : 0);
      __threadfence_system();
      for (int r = 0; r < pp.n; ++r)
        if (r != pp.rank) st_release_sys_i(pp.flags[r] + pp.rank, epoch);
    }
  }
}

// Barrier over the group: raise flags[r][rank] = epoch at every rank, wait for all of mine.
__global__ void group_barrier_kernel(const PeerPtrs pp) {
  const int epoch = pp.epoch + (pp.epoch_base ? *pp.epoch_base : 0);
  const int r = threadIdx.x;
  if (r < pp.n && TP_CHECK(pp.n <= kMaxDp && pp.rank >= 0 && pp.rank < pp.n, pp.err, kErrCheckPeer)) {
    __threadfence_system();
    st_release_sys_i(pp.flags[r] + pp.rank, epoch);
    spin_until(pp.flags[pp.rank] + r, epoch, pp.err, kErrWaitPeer);
  }
}

// out[i] += sum over ranks r of ptr[r][i], i < n (fp32; peer loads).
__global__ void __launch_bounds__(256) peer_sum_kernel(float* __restrict__ out, int n, const PeerPtrs pp) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float t = 0.0f;
  for (int r = 0; r < pp.n; ++r) t += __ldcg(static_cast<const float*>(pp.ptr[r]) + i);
  out[i] += t;
}

static bool make_peer_ptrs(PeerPtrs* pp, void* const* ptrs, int* const* flag_ptrs, int n, int rank,
                           int epoch, const int* epoch_base, int* counter, int* err) {
  if (n < 1 || n > kMaxDp || rank < 0 || rank >= n) return false;
  for (int i = 0; i < kMaxDp; ++i) {
    pp->ptr[i] = (ptrs && i < n) ? ptrs[i] : nullptr;
    pp->flags[i] = (flag_ptrs && i < n) ? flag_ptrs[i] : nullptr;
  }
  pp->n = n; pp->rank = rank; pp->epoch = epoch; pp->epoch_base = epoch_base; pp->counter = counter;
  pp->err = err;
  return true;
}

}  // namespace tp

// All-gather by push: `bytes` (a multiple of 16) at `src` in this rank's buffer go to dst_ptrs[r]
// for every other rank r, then flag_ptrs[r][rank] = epoch + *epoch_base.  Consumer: tp_gemm_ag.
extern "C" int tp_ag_push(const void* src, long long bytes, void* const* dst_ptrs, int* const* flag_ptrs,
                          int n, int rank, int epoch, const int* epoch_base, int* counter, void* stream) {
  if (bytes <= 0 || bytes % 16 || !dst_ptrs || !flag_ptrs || !counter) return kErrBadArgument;
  PeerPtrs pp;
  if (!make_peer_ptrs(&pp, dst_ptrs, flag_ptrs, n, rank, epoch, epoch_base, counter, nullptr))
    return kErrBadArgument;
  const long long n_vec = bytes / 16;
  long long blocks = (n_vec + 255) / 256;
  if (blocks > 2ll * num_sms()) blocks = 2ll * num_sms();
  ag_push_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), n_vec, pp);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

namespace tp {
__global__ void ag_signal_kernel(const PeerPtrs pp) {
  const int r = threadIdx.x;
  if (r < pp.n && r != pp.rank &&
      TP_CHECK(pp.n <= kMaxDp && pp.rank >= 0 && pp.rank < pp.n, pp.err, kErrCheckPeer)) {
    const int epoch = pp.epoch + (pp.epoch_base ? *pp.epoch_base : 0);
    __threadfence_system();
    st_release_sys_i(pp.flags[r] + pp.rank, epoch);
  }
}
}  // namespace tp

// All-gather by copy engine: `bytes` at `src` (this rank's shard, already in its final place in
// the local buffer) are copied to dst_ptrs[r] for every other rank r with one cudaMemcpyAsync per
// peer, then a one-warp kernel raises flag_ptrs[r][rank] = epoch + *epoch_base at every peer.  No SM
// time is spent on the transfer, so it can run on a side stream underneath the consumer
// (tp_gemm_ag), which starts with the row blocks of its own rank.
extern "C" int tp_ag_copy(const void* src, long long bytes, void* const* dst_ptrs, int* const* flag_ptrs,
                          int n, int rank, int epoch, const int* epoch_base, void* stream) {
  if (bytes <= 0 || !dst_ptrs || !flag_ptrs) return kErrBadArgument;
  PeerPtrs pp;
  if (!make_peer_ptrs(&pp, dst_ptrs, flag_ptrs, n, rank, epoch, epoch_base, nullptr, nullptr))
    return kErrBadArgument;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  for (int r = 0; r < n; ++r) {
    if (r == rank) continue;
    if (cudaMemcpyAsync(dst_ptrs[r], src, static_cast<size_t>(bytes), cudaMemcpyDefault, s) != cudaSuccess)
      return kErrDriver;
  }
  ag_signal_kernel<<<1, 32, 0, s>>>(pp);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

// Device-side barrier of a tensor-parallel group between steps: flag_ptrs[r] is rank r's barrier
// flag array (n ints), epoch + *epoch_base must grow from call to call.  A wait that runs out
// writes kErrWaitPeer to *err.
extern "C" int tp_group_barrier(int* const* flag_ptrs, int n, int rank, int epoch, const int* epoch_base,
                                int* err, void* stream) {
  if (!flag_ptrs) return kErrBadArgument;
  PeerPtrs pp;
  if (!make_peer_ptrs(&pp, nullptr, flag_ptrs, n, rank, epoch, epoch_base, nullptr, err))
    return kErrBadArgument;
  group_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pp);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

// out[i] += sum_r src_ptrs[r][i] for i < n floats (src_ptrs[r]: the same region of every rank's
// peer-mapped buffer, complete on every rank: call tp_group_barrier first).
extern "C" int tp_peer_sum(float* out, int n, void* const* src_ptrs, int n_ranks, int rank, void* stream) {
  if (n <= 0 || !src_ptrs) return kErrBadArgument;
  PeerPtrs pp;
  if (!make_peer_ptrs(&pp, src_ptrs, nullptr, n_ranks, rank, 0, nullptr, nullptr, nullptr))
    return kErrBadArgument;
  peer_sum_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(out, n, pp);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

// Limit of every bounded device-side wait of this library (mbarrier, peer flags), on the current
// device; the default is 5 s.  Call it with no kernel of the library in flight.
TP_DEFINE_WAIT_LIMIT_SETTER(tp_set_wait_limit_ns_comm)
extern "C" int tp_set_wait_limit_ns_gemm(unsigned long long ns);
extern "C" int tp_set_wait_limit_ns_attn(unsigned long long ns);
extern "C" int tp_set_wait_limit_ns(unsigned long long ns) {
  if (ns == 0) return kErrBadArgument;
  if (cudaDeviceSynchronize() != cudaSuccess) return kErrDriver;
  const int a = tp_set_wait_limit_ns_comm(ns), b = tp_set_wait_limit_ns_gemm(ns),
            c = tp_set_wait_limit_ns_attn(ns);
  return (a | b | c) ? kErrDriver : kOk;
}

// Which build this is: 1 when the kernels carry their index checks (-DTP_CHECKED), else 0.
extern "C" int tp_checked_build(void) {
#ifdef TP_CHECKED
  return 1;
#else
  return 0;
#endif
}

namespace tp {
__global__ void checked_selftest_kernel(int value, int limit, int* err) {
  if (TP_CHECK(value >= 0 && value < limit, err, kErrCheckSelfTest)) return;
}
}  // namespace tp

// Runs the check `0 <= value < limit` inside a kernel, the way the kernels check their indices.
// Checked build: a failing check leaves kErrCheckSelfTest in *err (nothing traps, nothing is
// accessed).  Regular build: the check is compiled out and *err is never written.
extern "C" int tp_checked_selftest(int value, int limit, int* err, void* stream) {
  if (!err) return kErrBadArgument;
  tp::checked_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(value, limit, err);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}
