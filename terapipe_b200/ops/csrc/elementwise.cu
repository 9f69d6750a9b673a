// Memory-bound kernels of the training step: LayerNorm forward/backward, bias-gradient
// column sums, the fused mixed-precision Adam update and small helpers.  All use 16-byte
// vector accesses; statistics and reductions are fp32.
#include "common.cuh"
#include "ptx.cuh"

namespace tp {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Output fan-out of the LayerNorm kernels under sequence-parallel tensor parallelism: the kernel
// runs on this rank's token shard and stores each output row at the same offset into the buffer
// of EVERY rank of the group (dst[0..n); plain peer stores over NVLink for the others), which is
// the all-gather the following column-parallel GEMM needs.  When all CTAs are done, the last one
// raises flags[r][rank] = epoch + *epoch_base at every other rank r; the consumer (tp_gemm_ag)
// waits for that value.  n == 1 and flags unset: an ordinary single-destination kernel.
constexpr int kMaxPush = 8;
struct PushDst {
  void* dst[kMaxPush];
  int* flags[kMaxPush];
  int n, rank, epoch;
  const int* epoch_base;
  int* counter;   // zero between launches; counts finished CTAs
};

__device__ __forceinline__ void push_signal(const PushDst& pd) {
  if (pd.n <= 1 || pd.counter == nullptr) return;
  __threadfence_system();   // this thread's peer stores are visible system-wide
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned total = gridDim.x * gridDim.y;
    if (atomicAdd(reinterpret_cast<unsigned*>(pd.counter), 1u) == total - 1) {
      *pd.counter = 0;
      const int epoch = pd.epoch + (pd.epoch_base ? *pd.epoch_base : 0);
      __threadfence_system();
      for (int r = 0; r < pd.n; ++r)
        if (r != pd.rank)
          asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(pd.flags[r] + pd.rank), "r"(epoch) : "memory");
    }
  }
}

// Sum over the CTA; every thread gets the result.  `red` holds >= 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

template <typename T> __device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = Elem<T>::unpack2(w[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}
template <typename T> __device__ __forceinline__ void load8(const T* p, float (&f)[8]) {
  unpack8<T>(*reinterpret_cast<const uint4*>(p), f);
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float (&f)[8]) {
  uint4 u;
  u.x = Elem<T>::pack2(f[0], f[1]);
  u.y = Elem<T>::pack2(f[2], f[3]);
  u.z = Elem<T>::pack2(f[4], f[5]);
  u.w = Elem<T>::pack2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// ------------------------------------------------------------------ LayerNorm
// A row is handled by WPR warps; each lane keeps NV vectors of 8 consecutive elements, vector i
// of lane l of warp w at column ((i * WPR + w) * 32 + l) * 8, so a warp reads 512 contiguous
// bytes per vector.  A CTA of 8 warps (16 when WPR = 16) holds RPC = max(1, 8 / WPR) rows.
template <int WPR> struct LnGeom {
  static constexpr int kWarps = WPR > 8 ? WPR : 8;
  static constexpr int kRowsPerCta = kWarps / WPR;
  static constexpr int kThreads = kWarps * 32;
};

// Sum over the WPR warps of a row group; `red` is [slots][RPC][WPR] (ping-pong by `slot`).  Only
// the warps of the group meet (named barrier 1 + grp), so the row groups of a CTA run
// independently.  RPC = row groups per CTA (at most 15 named barriers are free).
template <int WPR, int RPC>
__device__ __forceinline__ float group_sum_named(float v, float* red, int slot, int grp, int wr, int lane) {
  v = warp_sum(v);
  if (WPR == 1) return v;
  float* r = red + (slot * RPC + grp) * WPR;
  if (lane == 0) r[wr] = v;
  asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(WPR * 32) : "memory");
  float t = 0.0f;
#pragma unroll
  for (int i = 0; i < WPR; ++i) t += r[i];
  return t;
}

template <typename T, int NV, int WPR>
__global__ void __launch_bounds__(LnGeom<WPR>::kThreads)
layernorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gamma,
                     const T* __restrict__ beta, const PushDst pd, float* __restrict__ mean_out,
                     float* __restrict__ rstd_out, int rows, int H, float eps) {
  using G = LnGeom<WPR>;
  __shared__ float red[2 * G::kRowsPerCta * WPR + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int grp = warp / WPR, wr = warp % WPR;
  pdl_wait();
  const long long row = static_cast<long long>(blockIdx.x) * G::kRowsPerCta + grp;
  const bool row_ok = row < rows;
  float v[NV][8];
  uint4 gq[NV], bq[NV];   // gamma / beta of this lane's columns, fetched with the row (16-bit, packed)
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = ((i * WPR + wr) * 32 + lane) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) v[i][j] = 0.0f;
    gq[i] = make_uint4(0, 0, 0, 0);
    bq[i] = make_uint4(0, 0, 0, 0);
    if (row_ok && col < H) {
      load8(x + row * H + col, v[i]);
      gq[i] = *reinterpret_cast<const uint4*>(gamma + col);
      bq[i] = *reinterpret_cast<const uint4*>(beta + col);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += v[i][j];
    }
  }
  const float mean = group_sum_named<WPR, G::kRowsPerCta>(s, red, 0, grp, wr, lane) / H;
  float q = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = ((i * WPR + wr) * 32 + lane) * 8;
    if (col < H) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = v[i][j] - mean;
        q += d * d;
      }
    }
  }
  const float rstd = rsqrtf(group_sum_named<WPR, G::kRowsPerCta>(q, red, 1, grp, wr, lane) / H + eps);
  if (row_ok) {
    if (wr == 0 && lane == 0) {
      mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int col = ((i * WPR + wr) * 32 + lane) * 8;
      if (col < H) {
        float g[8], b[8], o[8];
        unpack8<T>(gq[i], g);
        unpack8<T>(bq[i], b);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mean) * rstd * g[j] + b[j];
        for (int d = 0; d < pd.n; ++d) store8(static_cast<T*>(pd.dst[d]) + row * H + col, o);
      }
    }
  }
  push_signal(pd);
}

// Backward geometry: 16 warps per CTA, so a CTA holds 16 / WPR rows at a time (8 rows of 2048
// columns; one CTA per SM then covers 1184 rows, a whole 1024-row token slice, in one pass).
template <int WPR> struct LnBwdGeom {
  static constexpr int kWarps = 16;
  static constexpr int kRowsPerCta = kWarps / WPR;
  static constexpr int kThreads = kWarps * 32;
};

// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)) (+ dres), g = dy * gamma.
// Persistent CTAs stride over rows.  The partial sums of dgamma = sum dy*xhat and dbeta = sum dy
// live in shared memory, one [2][H] region per row group, each lane adding to its own columns
// (no synchronisation inside the loop, and no accumulator registers: 512 threads fit).  Inside a
// region the two 16-byte halves of a lane's 8 columns lie in two planes, [array][half][H / 8][4],
// so that neighbouring lanes touch neighbouring 16 bytes (no bank conflicts).  At the end the regions are added in a fixed order and the CTA writes (or adds to) one
// slot of scratch[gridDim.x][2][H]; a second kernel adds the slots into the fp32 gradients.
template <typename T, int NV, int WPR>
__global__ void __launch_bounds__(LnBwdGeom<WPR>::kThreads, 1)
layernorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                     const float* __restrict__ mean, const float* __restrict__ rstd,
                     const T* __restrict__ gamma, const T* __restrict__ dres, const PushDst pd,
                     float* __restrict__ scratch, int rows, int H, int accumulate_slots) {
  using G = LnBwdGeom<WPR>;
  extern __shared__ __align__(16) float part_smem[];  // [kRowsPerCta][2][H]
  __shared__ float red[2 * 2 * G::kRowsPerCta * WPR + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int grp = warp / WPR, wr = warp % WPR;
  float* my_part = part_smem + static_cast<long long>(grp) * 2 * H;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = ((i * WPR + wr) * 32 + lane) * 8;
    if (col < H) {
      const float4 z = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      float4* sgam = reinterpret_cast<float4*>(my_part + (col >> 1));
      float4* sbet = reinterpret_cast<float4*>(my_part + H + (col >> 1));
      sgam[0] = z; sgam[H >> 3] = z; sbet[0] = z; sbet[H >> 3] = z;
    }
  }
  pdl_wait();
  int parity = 0;
  for (long long base = static_cast<long long>(blockIdx.x) * G::kRowsPerCta; base < rows;
       base += static_cast<long long>(gridDim.x) * G::kRowsPerCta, parity ^= 1) {
    const long long row = base + grp;
    const bool row_ok = row < rows;
    const float mu = row_ok ? mean[row] : 0.0f, rs = row_ok ? rstd[row] : 0.0f;
    float xh[NV][8], g[NV][8];
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int col = ((i * WPR + wr) * 32 + lane) * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) { xh[i][j] = 0.0f; g[i][j] = 0.0f; }
      if (row_ok && col < H) {
        float xv[8], dyv[8], gam[8];
        load8(x + row * H + col, xv);
        load8(dy + row * H + col, dyv);
        load8(gamma + col, gam);
        float4* sgam = reinterpret_cast<float4*>(my_part + (col >> 1));      // half 0; half 1 is
        float4* sbet = reinterpret_cast<float4*>(my_part + H + (col >> 1));  // H / 2 floats further
        float pg[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xv[j] - mu) * rs;
          g[i][j] = dyv[j] * gam[j];
          s1 += g[i][j];
          s2 += g[i][j] * xh[i][j];
          pg[j] = dyv[j] * xh[i][j];
        }
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf) {
          float4 a = sgam[hlf * (H >> 3)], c = sbet[hlf * (H >> 3)];
          a.x += pg[4 * hlf]; a.y += pg[4 * hlf + 1]; a.z += pg[4 * hlf + 2]; a.w += pg[4 * hlf + 3];
          c.x += dyv[4 * hlf]; c.y += dyv[4 * hlf + 1]; c.z += dyv[4 * hlf + 2]; c.w += dyv[4 * hlf + 3];
          sgam[hlf * (H >> 3)] = a;
          sbet[hlf * (H >> 3)] = c;
        }
      }
    }
    const float m1 = group_sum_named<WPR, G::kRowsPerCta>(s1, red, 2 * parity, grp, wr, lane) / H;
    const float m2 = group_sum_named<WPR, G::kRowsPerCta>(s2, red, 2 * parity + 1, grp, wr, lane) / H;
    if (row_ok) {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int col = ((i * WPR + wr) * 32 + lane) * 8;
        if (col < H) {
          float o[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = rs * (g[i][j] - m1 - xh[i][j] * m2);
          if (dres) {
            float r[8];
            load8(dres + row * H + col, r);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] += r[j];
          }
          for (int d = 0; d < pd.n; ++d) store8(static_cast<T*>(pd.dst[d]) + row * H + col, o);
        }
      }
    }
  }
  // add the row groups' regions in a fixed order (16-byte accesses), then write the CTA's sums
  // to (or add them into) its slot of the persistent partial buffer
  __syncthreads();
  float* sg = scratch + static_cast<long long>(blockIdx.x) * 2 * H;
  for (int c = threadIdx.x * 4; c < 2 * H; c += blockDim.x * 4) {
    // columns [q, q + 4) of array c / H: half (q / 4) & 1 of the 8-column group q / 8
    const int arr = c >= H ? 1 : 0, q = c - arr * H;
    const int sidx = arr * H + ((q >> 2) & 1) * (H >> 1) + (q >> 3) * 4;
    float4 v = *reinterpret_cast<const float4*>(part_smem + sidx);
#pragma unroll
    for (int gsel = 1; gsel < G::kRowsPerCta; ++gsel) {
      const float4 o = *reinterpret_cast<const float4*>(part_smem + static_cast<long long>(gsel) * 2 * H + sidx);
      v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
    }
    if (accumulate_slots) {
      const float4 o = __ldcg(reinterpret_cast<const float4*>(sg + c));
      v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
    }
    __stcg(reinterpret_cast<float4*>(sg + c), v);
  }
  push_signal(pd);
}

// dgamma[c] += sum_p scratch[p][0][c]; dbeta[c] += sum_p scratch[p][1][c]; optionally clears the
// slots afterwards.  blockDim = (32, 8): 32 columns per CTA, 8 lanes over the slots (4 loads in
// flight per thread), fixed-order tree in shared memory.
// clear bit 0: zero the slots afterwards; bit 1: overwrite dgamma/dbeta instead of adding.
__global__ void layernorm_bwd_reduce_kernel(float* __restrict__ scratch, int parts, int H,
                                            float* __restrict__ dgamma, float* __restrict__ dbeta,
                                            int clear) {
  __shared__ float sm[8][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  const long long stride = 2ll * H;
  float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
  if (c < 2 * H) {
    int p = threadIdx.y;
    for (; p + 24 < parts; p += 32) {
      s0 += __ldcg(scratch + p * stride + c);
      s1 += __ldcg(scratch + (p + 8) * stride + c);
      s2 += __ldcg(scratch + (p + 16) * stride + c);
      s3 += __ldcg(scratch + (p + 24) * stride + c);
    }
    for (; p < parts; p += 8) s0 += __ldcg(scratch + p * stride + c);
    if (clear & 1)
      for (int q = threadIdx.y; q < parts; q += 8) scratch[q * stride + c] = 0.0f;
  }
  sm[threadIdx.y][threadIdx.x] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (threadIdx.y == 0 && c < 2 * H) {
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += sm[i][threadIdx.x];
    if (clear & 2) {
      if (c < H) dgamma[c] = t;
      else dbeta[c - H] = t;
    } else {
      if (c < H) dgamma[c] += t;
      else dbeta[c - H] += t;
    }
  }
}

// ------------------------------------------------------------------ bias gradient
// db[n] += sum_rows dy[row][n]; blockDim = (32, 16): 32 vectors of 8 columns, 16 row lanes.
template <typename T>
__global__ void colsum_kernel(const T* __restrict__ dy, long long ld, int rows, int N,
                              float* __restrict__ db) {
  __shared__ float sm[16][32][8 + 1];
  const int col = (blockIdx.x * 32 + threadIdx.x) * 8;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (col < N) {
    for (int r = blockIdx.y * 16 + threadIdx.y; r < rows; r += 16 * gridDim.y) {
      float v[8];
      load8(dy + static_cast<long long>(r) * ld + col, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) sm[threadIdx.y][threadIdx.x][j] = acc[j];
  __syncthreads();
  if (threadIdx.y < 8) {
    // thread (x, y<8) finishes column col + y
    float s = 0.0f;
#pragma unroll
    for (int r = 0; r < 16; ++r) s += sm[r][threadIdx.x][threadIdx.y];
    if (col + threadIdx.y < N) {
      if (gridDim.y == 1) db[col + threadIdx.y] += s;
      else atomicAdd(&db[col + threadIdx.y], s);
    }
  }
}

// ------------------------------------------------------------------ fused Adam
// state[0] = step count (as float), state[1] = 1 - beta1^t, state[2] = 1 - beta2^t.
__global__ void adam_tick_kernel(float* state, float beta1, float beta2) {
  const float t = state[0] + 1.0f;
  state[0] = t;
  state[1] = 1.0f - powf(beta1, t);
  state[2] = 1.0f - powf(beta2, t);
}

// One pass over flat buffers: g = grad * grad_scale; m, v, p (fp32 master) updated in place;
// the 16-bit model copy is rewritten and the gradient accumulator is zeroed.
template <typename T>
__global__ void fused_adam_kernel(float* __restrict__ grad, float* __restrict__ p,
                                  float* __restrict__ m, float* __restrict__ v,
                                  T* __restrict__ model, long long n4, const float* __restrict__ state,
                                  float lr, float beta1, float beta2, float eps, float weight_decay,
                                  float grad_scale) {
  const float bc1 = state[1], bc2 = state[2];
  const float inv_bc2_sqrt = rsqrtf(bc2);
  const float step = lr / bc1;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 g4 = reinterpret_cast<float4*>(grad)[i];
    float4 p4 = reinterpret_cast<float4*>(p)[i];
    float4 m4 = reinterpret_cast<float4*>(m)[i];
    float4 v4 = reinterpret_cast<float4*>(v)[i];
    float* g = reinterpret_cast<float*>(&g4);
    float* pp = reinterpret_cast<float*>(&p4);
    float* mm = reinterpret_cast<float*>(&m4);
    float* vv = reinterpret_cast<float*>(&v4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = g[j] * grad_scale;
      mm[j] = beta1 * mm[j] + (1.0f - beta1) * gj;
      vv[j] = beta2 * vv[j] + (1.0f - beta2) * gj * gj;
      const float denom = sqrtf(vv[j]) * inv_bc2_sqrt + eps;
      pp[j] = pp[j] - step * (mm[j] / denom) - lr * weight_decay * pp[j];
    }
    reinterpret_cast<float4*>(p)[i] = p4;
    reinterpret_cast<float4*>(m)[i] = m4;
    reinterpret_cast<float4*>(v)[i] = v4;
    reinterpret_cast<float4*>(grad)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    uint2 o;
    o.x = Elem<T>::pack2(pp[0], pp[1]);
    o.y = Elem<T>::pack2(pp[2], pp[3]);
    reinterpret_cast<uint2*>(model)[i] = o;
  }
}

template <typename T>
__global__ void fill_kernel(T* p, long long n, float value) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    p[i] = Elem<T>::from_f(value);
}

}  // namespace tp

using namespace tp;

// Geometry: the smallest power-of-two warps-per-row (<= 16) that keeps at most 4 vectors of 8
// elements per lane.
static inline bool ln_geometry(int H, int* nv, int* wpr) {
  if (H % 8 || H <= 0) return false;
  const int vecs = H / 8;
  for (int w = 1; w <= 16; w *= 2) {
    const int n = (vecs + 32 * w - 1) / (32 * w);
    if (n <= 4) { *nv = n; *wpr = w; return true; }
  }
  return false;
}

#define TP_LN_DISPATCH_WPR(T, NV, CALL)                  \
  switch (wpr) {                                          \
    case 1: CALL(T, NV, 1); break;                        \
    case 2: CALL(T, NV, 2); break;                        \
    case 4: CALL(T, NV, 4); break;                        \
    case 8: CALL(T, NV, 8); break;                        \
    default: CALL(T, NV, 16); break;                      \
  }
#define TP_LN_DISPATCH(T, CALL)                           \
  switch (nv) {                                           \
    case 1: TP_LN_DISPATCH_WPR(T, 1, CALL) break;         \
    case 2: TP_LN_DISPATCH_WPR(T, 2, CALL) break;         \
    case 3: TP_LN_DISPATCH_WPR(T, 3, CALL) break;         \
    default: TP_LN_DISPATCH_WPR(T, 4, CALL) break;        \
  }

namespace tp {
static PushDst single_dst(void* y) {
  PushDst pd;
  for (int i = 0; i < kMaxPush; ++i) { pd.dst[i] = nullptr; pd.flags[i] = nullptr; }
  pd.dst[0] = y;
  pd.n = 1; pd.rank = 0; pd.epoch = 0; pd.epoch_base = nullptr; pd.counter = nullptr;
  return pd;
}

static bool make_push(PushDst* pd, void* const* dst_ptrs, int* const* flag_ptrs, int n, int rank,
                      int epoch, const int* epoch_base, int* counter) {
  if (n < 1 || n > kMaxPush || rank < 0 || rank >= n || !dst_ptrs || !flag_ptrs || !counter) return false;
  for (int i = 0; i < kMaxPush; ++i) {
    pd->dst[i] = i < n ? dst_ptrs[i] : nullptr;
    pd->flags[i] = i < n ? flag_ptrs[i] : nullptr;
  }
  pd->n = n; pd->rank = rank; pd->epoch = epoch; pd->epoch_base = epoch_base; pd->counter = counter;
  return true;
}

static int layernorm_fwd_launch(int dtype, const void* x, const void* gamma, const void* beta,
                                const PushDst& pd, float* mean, float* rstd, int rows, int H,
                                float eps, cudaStream_t s) {
  if (rows <= 0) return kOk;
  int nv, wpr;
  if (!ln_geometry(H, &nv, &wpr)) return kErrBadArgument;
#define LN_FWD(T, NV, WPR)                                                                       \
  launch_pdl(layernorm_fwd_kernel<T, NV, WPR>,                                                   \
             dim3((rows + LnGeom<WPR>::kRowsPerCta - 1) / LnGeom<WPR>::kRowsPerCta),             \
             dim3(LnGeom<WPR>::kThreads), 0, s, 1, static_cast<const T*>(x),                     \
             static_cast<const T*>(gamma), static_cast<const T*>(beta), pd, mean, rstd, rows, H, eps)
  if (dtype == 1) { TP_LN_DISPATCH(__nv_bfloat16, LN_FWD) }
  else { TP_LN_DISPATCH(__half, LN_FWD) }
#undef LN_FWD
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}
}  // namespace tp

extern "C" int tp_layernorm_fwd(int dtype, const void* x, const void* gamma, const void* beta,
                                void* y, float* mean, float* rstd, int rows, int H, float eps,
                                void* stream) {
  return layernorm_fwd_launch(dtype, x, gamma, beta, single_dst(y), mean, rstd, rows, H, eps,
                              static_cast<cudaStream_t>(stream));
}

// LayerNorm forward of this rank's token shard whose output rows go to the same place in the
// buffer of every rank of a tensor-parallel group (`y_ptrs[r]`, r < n; entry `rank` is the local
// buffer), followed by a flag at every peer: flag_ptrs[r][rank] = epoch + *epoch_base.
// `counter` is a zero-initialised device int used to find the last CTA.  The consumer is
// tp_gemm_ag with the same epoch.
extern "C" int tp_layernorm_fwd_push(int dtype, const void* x, const void* gamma, const void* beta,
                                     void* const* y_ptrs, float* mean, float* rstd, int rows, int H,
                                     float eps, int n, int rank, int* const* flag_ptrs, int epoch,
                                     const int* epoch_base, int* counter, void* stream) {
  PushDst pd;
  if (!make_push(&pd, y_ptrs, flag_ptrs, n, rank, epoch, epoch_base, counter)) return kErrBadArgument;
  return layernorm_fwd_launch(dtype, x, gamma, beta, pd, mean, rstd, rows, H, eps,
                              static_cast<cudaStream_t>(stream));
}

// Number of CTA slots the backward writes; scratch must hold parts * 2 * H floats.
extern "C" int tp_layernorm_bwd_parts(int rows) {
  const int cap = num_sms();
  return rows < cap ? rows : cap;
}

namespace tp {
// Opt the kernel in to more than 48 KB of shared memory, once per instantiation (the first,
// eager launch; never inside a stream capture).
template <typename K> static void ln_allow_smem(K kern) {
  // (instantiations of one element type share the function-pointer type K, so the kernels
  // already handled are remembered by address)
  static const void* seen[64];
  static int n_seen = 0;
  const void* key = reinterpret_cast<const void*>(kern);
  for (int i = 0; i < n_seen; ++i)
    if (seen[i] == key) return;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024);
  if (n_seen < 64) seen[n_seen++] = key;
}

static int ln_parts(int rows, int wpr) {
  const int rpc = 16 / wpr;   // LnBwdGeom<WPR>::kRowsPerCta
  int parts = (rows + rpc - 1) / rpc;
  const int cap = tp_layernorm_bwd_parts(rows);
  return parts > cap ? cap : parts;
}

// mode 0: write the CTA partials into `scratch` and fold them into dgamma/dbeta right away.
// mode 1: ADD the CTA partials into the persistent slots `scratch` (zero-initialised by the
//         caller) and leave dgamma/dbeta alone; tp_layernorm_bwd_finish folds them later.
static int layernorm_bwd_launch(int dtype, const void* dy, const void* x, const float* mean,
                                const float* rstd, const void* gamma, const void* dres,
                                const PushDst& pd, float* dgamma, float* dbeta, float* scratch,
                                int rows, int H, int mode, cudaStream_t s) {
  if (rows <= 0) return kOk;
  int nv, wpr;
  if (!ln_geometry(H, &nv, &wpr)) return kErrBadArgument;
  const int parts = ln_parts(rows, wpr);
  // one [2][H] fp32 region per row group of the CTA: at most 128 KB (H <= 1024 * WPR)
  const size_t smem = static_cast<size_t>(16 / wpr) * 2 * H * sizeof(float);
#define LN_BWD(T, NV, WPR)                                                                      \
  {                                                                                             \
    auto kern = layernorm_bwd_kernel<T, NV, WPR>;                                               \
    if (smem > 40 * 1024) ln_allow_smem(kern); /* dynamic + static must stay under 48 KB */    \
    launch_pdl(kern, dim3(parts), dim3(LnBwdGeom<WPR>::kThreads), smem, s, 1,                   \
               static_cast<const T*>(dy), static_cast<const T*>(x), mean, rstd,                 \
               static_cast<const T*>(gamma), static_cast<const T*>(dres), pd, scratch,           \
               rows, H, mode);                                                                  \
  }
  if (dtype == 1) { TP_LN_DISPATCH(__nv_bfloat16, LN_BWD) }
  else { TP_LN_DISPATCH(__half, LN_BWD) }
#undef LN_BWD
  if (mode == 0)
    layernorm_bwd_reduce_kernel<<<(2 * H + 31) / 32, dim3(32, 8), 0, s>>>(scratch, parts, H, dgamma,
                                                                          dbeta, 0);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}
}  // namespace tp

extern "C" int tp_layernorm_bwd(int dtype, const void* dy, const void* x, const float* mean,
                                const float* rstd, const void* gamma, const void* dres, void* dx,
                                float* dgamma, float* dbeta, float* scratch, int rows, int H,
                                void* stream) {
  return layernorm_bwd_launch(dtype, dy, x, mean, rstd, gamma, dres, single_dst(dx), dgamma, dbeta,
                              scratch, rows, H, 0, static_cast<cudaStream_t>(stream));
}

// Variant that only accumulates into persistent partial slots (tp_layernorm_bwd_parts(rows)
// slots of 2*H floats, zero before the first call of a backward pass).
extern "C" int tp_layernorm_bwd_accum(int dtype, const void* dy, const void* x, const float* mean,
                                      const float* rstd, const void* gamma, const void* dres,
                                      void* dx, float* slots, int rows, int H, void* stream) {
  return layernorm_bwd_launch(dtype, dy, x, mean, rstd, gamma, dres, single_dst(dx), nullptr, nullptr,
                              slots, rows, H, 1, static_cast<cudaStream_t>(stream));
}

// tp_layernorm_bwd_accum on this rank's token shard with the input gradient rows stored into the
// buffer of every rank of the group and a flag raised at every peer (see tp_layernorm_fwd_push).
extern "C" int tp_layernorm_bwd_accum_push(int dtype, const void* dy, const void* x, const float* mean,
                                           const float* rstd, const void* gamma, const void* dres,
                                           void* const* dx_ptrs, float* slots, int rows, int H, int n,
                                           int rank, int* const* flag_ptrs, int epoch,
                                           const int* epoch_base, int* counter, void* stream) {
  PushDst pd;
  if (!make_push(&pd, dx_ptrs, flag_ptrs, n, rank, epoch, epoch_base, counter)) return kErrBadArgument;
  return layernorm_bwd_launch(dtype, dy, x, mean, rstd, gamma, dres, pd, nullptr, nullptr, slots, rows,
                              H, 1, static_cast<cudaStream_t>(stream));
}

// Fold `parts` slots into dgamma/dbeta (+=) and clear them for the next backward pass.
extern "C" int tp_layernorm_bwd_finish(float* slots, int parts, int H, float* dgamma, float* dbeta,
                                       void* stream) {
  layernorm_bwd_reduce_kernel<<<(2 * H + 31) / 32, dim3(32, 8), 0, static_cast<cudaStream_t>(stream)>>>(
      slots, parts, H, dgamma, dbeta, 1);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

// As tp_layernorm_bwd_finish, but dgamma/dbeta are overwritten with the folded sums (used when the
// sums of several ranks are added up afterwards, see tp_peer_sum).
extern "C" int tp_layernorm_bwd_finish_assign(float* slots, int parts, int H, float* dgamma,
                                              float* dbeta, void* stream) {
  layernorm_bwd_reduce_kernel<<<(2 * H + 31) / 32, dim3(32, 8), 0, static_cast<cudaStream_t>(stream)>>>(
      slots, parts, H, dgamma, dbeta, 3);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

extern "C" int tp_colsum(int dtype, const void* dy, long long ld, int rows, int N, float* db,
                         void* stream) {
  if (rows <= 0) return kOk;
  if (N % 8 || ld % 8) return kErrBadArgument;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 block(32, 16);
  int gy = rows / 256;
  gy = gy < 1 ? 1 : (gy > 8 ? 8 : gy);
  dim3 grid((N / 8 + 31) / 32, gy);
  if (dtype == 1)
    colsum_kernel<__nv_bfloat16><<<grid, block, 0, s>>>(static_cast<const __nv_bfloat16*>(dy), ld, rows, N, db);
  else
    colsum_kernel<__half><<<grid, block, 0, s>>>(static_cast<const __half*>(dy), ld, rows, N, db);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

extern "C" int tp_adam_tick(float* state, float beta1, float beta2, void* stream) {
  adam_tick_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(state, beta1, beta2);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

extern "C" int tp_fused_adam(int dtype, float* grad, float* p, float* m, float* v, void* model,
                             long long n, const float* state, float lr, float beta1, float beta2,
                             float eps, float weight_decay, float grad_scale, void* stream) {
  if (n % 4) return kErrBadArgument;
  if (n == 0) return kOk;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long n4 = n / 4;
  long long blocks = (n4 + 255) / 256;
  const long long cap = 8ll * num_sms();
  if (blocks > cap) blocks = cap;
  if (dtype == 1)
    fused_adam_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, s>>>(
        grad, p, m, v, static_cast<__nv_bfloat16*>(model), n4, state, lr, beta1, beta2, eps,
        weight_decay, grad_scale);
  else
    fused_adam_kernel<__half><<<static_cast<int>(blocks), 256, 0, s>>>(
        grad, p, m, v, static_cast<__half*>(model), n4, state, lr, beta1, beta2, eps, weight_decay,
        grad_scale);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

extern "C" int tp_fill(int dtype, void* p, long long n, float value, void* stream) {
  if (n <= 0) return kOk;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  long long blocks = (n + 255) / 256;
  if (blocks > 8ll * num_sms()) blocks = 8ll * num_sms();
  if (dtype == 1) fill_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, s>>>(static_cast<__nv_bfloat16*>(p), n, value);
  else fill_kernel<__half><<<static_cast<int>(blocks), 256, 0, s>>>(static_cast<__half*>(p), n, value);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

// ------------------------------------------------------------------ allocation-free variant
// LayerNorm backward for callers that cannot allocate: the per-CTA partial sums go to a fixed
// array inside the library image instead of a caller-provided buffer (see terapipe_noalloc.h).
#include "terapipe_noalloc.h"

namespace tp {
constexpr int kStaticSlots = 160;
constexpr int kStaticMaxH = 4096;
constexpr long long kStaticScratchFloats = static_cast<long long>(kStaticSlots) * 2 * kStaticMaxH;
// In host code this name is only a handle for cudaGetSymbolAddress; kernels get the address.
static __device__ __align__(256) float g_ln_static_scratch[kStaticScratchFloats];
}  // namespace tp

extern "C" long long tp_layernorm_bwd_noalloc_capacity(void) { return tp::kStaticScratchFloats; }

extern "C" int tp_layernorm_bwd_noalloc(int dtype, const void* dy, const void* x, const float* mean,
                                        const float* rstd, const void* gamma, const void* dres,
                                        void* dx, float* dgamma, float* dbeta, int rows, int H,
                                        void* stream) {
  constexpr int kMaxDevices = 64;
  static float* scratch_of_device[kMaxDevices] = {nullptr};
  if (rows <= 0) return kOk;
  if (H <= 0 || H % 8) return kErrBadArgument;
  if (H > kStaticMaxH) return kErrTooLarge;
  const int parts = tp_layernorm_bwd_parts(rows);
  if (static_cast<long long>(parts) * 2 * H > kStaticScratchFloats) return kErrTooLarge;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return kErrDriver;
  if (!scratch_of_device[dev]) {
    // once per device, with that device current: resolve the array's device address
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_ln_static_scratch) != cudaSuccess || !p) {
      cudaGetLastError();
      return kErrDriver;
    }
    scratch_of_device[dev] = p;
  }
  // mode 0 writes every slot it later reads, so stale contents of the shared array are harmless
  return layernorm_bwd_launch(dtype, dy, x, mean, rstd, gamma, dres, single_dst(dx), dgamma, dbeta,
                              scratch_of_device[dev], rows, H, 0, static_cast<cudaStream_t>(stream));
}

// Programmatic dependent launch of the GEMM, attention and LayerNorm kernels (off by default;
// TERAPIPE_PDL=1 in the environment or tp_set_pdl(1) turns it on).
extern "C" int tp_set_pdl(int enabled) {
  tp::pdl_enabled() = enabled ? 1 : 0;
  return kOk;
}
