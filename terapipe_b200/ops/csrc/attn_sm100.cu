// Slice-causal attention over a cached prefix for sm_100a (tcgen05 + TMEM + TMA).
//
// One token slice of `t` positions attends to the `c` positions cached by earlier slices plus
// itself; only the last `t` key columns carry a causal mask.  Q, K and V are read in place
// from the stage's full-length projection buffer
//     qkv[L][b][h][3][D]          (position, batch, local head, {q,k,v}, head dim)
// through 3-D tensor maps, so "appending to the KV cache" is just the QKV GEMM writing its
// rows; no gather/scatter kernels exist.  Scores never reach memory: S lives in TMEM, P is
// handed to the second MMA through shared memory, the running output stays in TMEM and is
// rescaled lazily (only when the row maximum grows by more than 2^8).
//
// Backward recomputes P from Q, K and the saved log-sum-exp (base 2); see the comment above
// attn_bwd_kernel.  No gradient accumulator crosses slices: the backward pass walks the
// slices in reverse, so when slice j is processed the attention-output gradients dO of all
// later slices already sit in a full-length buffer, and dK/dV of slice j's keys are computed
// in one go by streaming over those later queries.
//
// Forward CTA = 5 warps: warps 0..3 own one TMEM lane quarter each (one row per thread: softmax
// needs no shuffles), warp 4 elects one thread that issues all TMA copies and MMAs.
#include <math.h>
#include <string.h>

#include "common.cuh"
#include "ptx.cuh"

namespace tp {

constexpr int kAttnThreads = 160;

struct AttnParams {
  int t, c, b, h;
  float scale, scale2;  // d^-0.5 and d^-0.5 * log2(e)
  void* o;              // fwd out: [t*b][ld_o], column = head*D + e
  long long ld_o;
  float* lse2;          // [b*h][lse_stride], indexed by absolute position
  long long lse_stride;
  float* delta;         // bwd: [b*h][lse_stride] = rowsum(dO * O), indexed by absolute position
  int q_end;            // bwd: end (absolute position) of the rows already back-propagated
  void* dqkv;           // [t*b][ld_dqkv], same column order as qkv
  long long ld_dqkv;
  int* err;
};

// One arrival per warp (after the warp's lanes have finished their part): far cheaper than 32
// contending shared-memory atomics on the same barrier word.
__device__ __forceinline__ void warp_arrive(uint64_t* bar) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}

__device__ __forceinline__ void named_bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// Write one row (64 values) of a [128 x 64] 16-bit operand tile in the 128B-swizzled
// K-major layout expected by the UMMA descriptors.
template <typename T>
__device__ __forceinline__ void store_row64(uint8_t* tile, int row, const float* v) {
#pragma unroll
  for (int ch = 0; ch < 8; ++ch) {
    uint4 u;
    u.x = Elem<T>::pack2(v[ch * 8 + 0], v[ch * 8 + 1]);
    u.y = Elem<T>::pack2(v[ch * 8 + 2], v[ch * 8 + 3]);
    u.z = Elem<T>::pack2(v[ch * 8 + 4], v[ch * 8 + 5]);
    u.w = Elem<T>::pack2(v[ch * 8 + 6], v[ch * 8 + 7]);
    *reinterpret_cast<uint4*>(tile + row * 128 + ((ch ^ (row & 7)) << 4)) = u;
  }
}

// D[tmem] (+)= A * B^T with both operands K-major, K = DH*64 split in DH sub-tiles.
template <int DH>
__device__ __forceinline__ void mma_kk(uint32_t tmem_d, uint32_t a_base, uint32_t a_sub,
                                       uint32_t b_base, uint32_t b_sub, uint32_t idesc) {
#pragma unroll
  for (int hh = 0; hh < DH; ++hh)
#pragma unroll
    for (int k = 0; k < 4; ++k)
      umma_f16(tmem_d, umma_desc_sw128(a_base + hh * a_sub + k * 32, 16, 1024),
               umma_desc_sw128(b_base + hh * b_sub + k * 32, 16, 1024), idesc,
               (hh | k) != 0 ? 1u : 0u);
}

// D[tmem] (+)= A[128 x 64, K-major] * B[64 (k) x N, N-major tile with 64-wide chunks b_sub apart]
__device__ __forceinline__ void mma_kn(uint32_t tmem_d, uint32_t a_base, uint32_t b_base,
                                       uint32_t b_sub, uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int k = 0; k < 4; ++k)
    umma_f16(tmem_d, umma_desc_sw128(a_base + k * 32, 16, 1024),
             umma_desc_sw128(b_base + k * 2048, b_sub, 1024), idesc,
             (accumulate || k != 0) ? 1u : 0u);
}

struct AttnShared {
  uint64_t bars[20];
  uint32_t tmem_slot;
  int abort_flag;
};

// ============================================================================ forward
// Software pipeline: K/V tiles sit in a 4-stage ring (the prefix is streamed from HBM, so
// loads must be issued several blocks ahead), the S accumulator and the P tile are double
// buffered, and the
// MMA thread issues S(j+1) = Q K(j+1)^T before it waits for the softmax of block j, so the
// tensor core computes the next scores while the 128 softmax threads work on the current ones.
template <typename T, int D>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV,
                const AttnParams p) {
  constexpr int DH = D / 64;
  constexpr int kQSub = 128 * 128, kKSub = 64 * 128;
  constexpr uint32_t kTmemCols = 256;
  constexpr int KS = 4;  // K/V ring depth
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + DH * kQSub;          // [KS][DH][kKSub]
  uint8_t* sV = sK + KS * DH * kKSub;     // [KS][DH][kKSub]
  uint8_t* sP = sV + KS * DH * kKSub;     // [2][128][128B]
  AttnShared* sh = reinterpret_cast<AttnShared*>(sP + 2 * 128 * 128);
  uint64_t* bar_q = &sh->bars[0];
  uint64_t* bar_k = &sh->bars[1];      // [KS]
  uint64_t* bar_v = &sh->bars[5];      // [KS]
  uint64_t* bar_s = &sh->bars[9];      // [2]
  uint64_t* bar_sfree = &sh->bars[11]; // [2]
  uint64_t* bar_p = &sh->bars[13];     // [2]
  uint64_t* bar_pv = &sh->bars[15];    // [2]

  const int warp = threadIdx.x >> 5;
  const WaitCtx wctx{&sh->abort_flag, p.err};
  const int q0 = blockIdx.x * 128;
  const int bh = blockIdx.y;
  const int bi = bh / p.h, hi = bh % p.h;
  const int q_hi = min(p.t, q0 + 128);
  const int nkb = (p.c + q_hi + 63) / 64;

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int i = 0; i < KS; ++i) {
      mbar_init(&bar_k[i], 1);
      mbar_init(&bar_v[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_s[i], 1);
      mbar_init(&bar_sfree[i], 4);
      mbar_init(&bar_p[i], 4);
      mbar_init(&bar_pv[i], 1);
    }
    sh->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 4) {
    tmem_alloc(&sh->tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();  // set-up done; from here on the predecessor's results are read
  const uint32_t tmem = sh->tmem_slot;
  const uint32_t tO = tmem + 128;   // S[0] at 0, S[1] at 64, O at 128

  if (warp == 4) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = umma_idesc_f16(Elem<T>::fmt, 0, 0, 128, 64);
      constexpr uint32_t idesc_pv = umma_idesc_f16(Elem<T>::fmt, 0, 1, 128, D);
      auto load_kv = [&](int j) {
        const int st = j % KS;
        mbar_expect_tx(&bar_k[st], DH * kKSub);
        for (int hh = 0; hh < DH; ++hh)
          tma_load_3d(sK + (st * DH + hh) * kKSub, &tmKV, &bar_k[st], D + hh * 64, bh, j * 64);
        mbar_expect_tx(&bar_v[st], DH * kKSub);
        for (int hh = 0; hh < DH; ++hh)
          tma_load_3d(sV + (st * DH + hh) * kKSub, &tmKV, &bar_v[st], 2 * D + hh * 64, bh, j * 64);
      };
      auto issue_s = [&](int j) -> bool {
        const int ks = j % KS, sb = j & 1;
        if (!mbar_wait(&bar_k[ks], (j / KS) & 1, wctx, kErrWaitAttn)) return false;
        if (!mbar_wait(&bar_sfree[sb], ((j >> 1) & 1) ^ 1, wctx, kErrWaitAttn)) return false;
        tc_fence_after();
        mma_kk<DH>(tmem + sb * 64, smem_u32(sQ), kQSub, smem_u32(sK + ks * DH * kKSub), kKSub, idesc_s);
        umma_commit(&bar_s[sb]);
        return true;
      };
      mbar_expect_tx(bar_q, DH * kQSub);
      for (int hh = 0; hh < DH; ++hh)
        tma_load_3d(sQ + hh * kQSub, &tmQ, bar_q, hh * 64, bh, p.c + q0);
      for (int j = 0; j < KS && j < nkb; ++j) load_kv(j);
      bool ok = mbar_wait(bar_q, 0, wctx, kErrWaitAttn);
      if (ok) ok = issue_s(0);
      for (int j = 0; j < nkb && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (j + 1 < nkb) ok = issue_s(j + 1);
        if (!ok) break;
        ok = mbar_wait(&bar_p[st], ph, wctx, kErrWaitAttn) &&
             mbar_wait(&bar_v[j % KS], (j / KS) & 1, wctx, kErrWaitAttn);
        if (!ok) break;
        tc_fence_after();
        mma_kn(tO, smem_u32(sP + st * 128 * 128), smem_u32(sV + (j % KS) * DH * kKSub), kKSub, idesc_pv, j > 0);
        umma_commit(&bar_pv[st]);
        if (j >= 1 && j - 1 + KS < nkb) {
          // ring stage (j-1) % KS is reusable once PV(j-1) has finished reading V(j-1); waiting
          // for the PREVIOUS block keeps this thread off the critical path of the current one
          ok = mbar_wait(&bar_pv[(j - 1) & 1], ((j - 1) >> 1) & 1, wctx, kErrWaitAttn);
          if (!ok) break;
          load_kv(j - 1 + KS);
        }
      }
    }
  } else {
    const int r = threadIdx.x;  // row of the tile = TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const int qi = q0 + r;
    const int qpos = p.c + qi;
    float m = -INFINITY, l = 0.0f;
    bool ok = true;
    for (int j = 0; j < nkb; ++j) {
      const int st = j & 1;
      ok = mbar_wait(&bar_s[st], (j >> 1) & 1, wctx, kErrWaitAttn);
      if (!ok) break;
      tc_fence_after();
      float s[64];
      {
        uint32_t r0[32], r1[32];
        __syncwarp();
        tmem_ld_32x32(tmem + st * 64 + lane_base, r0);
        tmem_ld_32x32(tmem + st * 64 + lane_base + 32, r1);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          s[i] = __uint_as_float(r0[i]);
          s[32 + i] = __uint_as_float(r1[i]);
        }
      }
      tc_fence_before();
      warp_arrive(&bar_sfree[st]);
      float mx = -INFINITY;
      const int kbase = j * 64;
      if (kbase + 63 <= p.c + q0) {   // every key of the block is visible to every row
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          s[i] *= p.scale2;
          mx = fmaxf(mx, s[i]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          s[i] = (kbase + i <= qpos) ? s[i] * p.scale2 : -INFINITY;
          mx = fmaxf(mx, s[i]);
        }
      }
      bool need = false;
      float alpha = 1.0f;
      if (j == 0) {
        m = mx;
      } else if (mx > m + 8.0f) {
        need = true;
        alpha = exp2f(m - mx);
        m = mx;
        l *= alpha;
      }
      if (__any_sync(0xffffffffu, need)) {
        // O may only be touched once PV(j-1) has been accumulated
        ok = mbar_wait(&bar_pv[(j - 1) & 1], ((j - 1) >> 1) & 1, wctx, kErrWaitAttn);
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int ch = 0; ch < D / 32; ++ch) {
          uint32_t raw[32];
          tmem_ld_32x32(tO + lane_base + ch * 32, raw);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) raw[i] = __float_as_uint(__uint_as_float(raw[i]) * alpha);
          tmem_st_32x32(tO + lane_base + ch * 32, raw);
        }
        tmem_st_wait();
      }
      float sum = 0.0f;
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        s[i] = exp2f(s[i] - m);
        sum += s[i];
      }
      l += sum;
      store_row64<T>(sP + st * 128 * 128, r, s);
      fence_proxy_async();
      tc_fence_before();
      warp_arrive(&bar_p[st]);
    }
    if (ok) ok = mbar_wait(&bar_pv[(nkb - 1) & 1], ((nkb - 1) >> 1) & 1, wctx, kErrWaitAttn);
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.0f / l;
      // checked build: the row's statistics slot and its columns of the output exist
      const bool row_ok = qi < p.t && TP_CHECK(qpos >= 0 && qpos < p.lse_stride && (hi + 1) * D <= p.ld_o,
                                               p.err, kErrCheckAttn);
      T* orow = static_cast<T*>(p.o) + (static_cast<long long>(qi) * p.b + bi) * p.ld_o + hi * D;
#pragma unroll 1
      for (int ch = 0; ch < D / 32; ++ch) {
        uint32_t raw[32];
        __syncwarp();
        tmem_ld_32x32(tO + lane_base + ch * 32, raw);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 u;
            u.x = Elem<T>::pack2(__uint_as_float(raw[g * 8 + 0]) * inv_l, __uint_as_float(raw[g * 8 + 1]) * inv_l);
            u.y = Elem<T>::pack2(__uint_as_float(raw[g * 8 + 2]) * inv_l, __uint_as_float(raw[g * 8 + 3]) * inv_l);
            u.z = Elem<T>::pack2(__uint_as_float(raw[g * 8 + 4]) * inv_l, __uint_as_float(raw[g * 8 + 5]) * inv_l);
            u.w = Elem<T>::pack2(__uint_as_float(raw[g * 8 + 6]) * inv_l, __uint_as_float(raw[g * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + ch * 32 + g * 8) = u;
          }
        }
      }
      if (row_ok) p.lse2[static_cast<long long>(bh) * p.lse_stride + qpos] = m + log2f(l);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (sh->abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_after();
  if (warp == 4) tmem_dealloc(tmem, kTmemCols);
}

// ============================================================================ delta = rowsum(dO * O)
template <typename T>
__global__ void attn_delta_kernel(const T* __restrict__ o, long long ld_o, const T* __restrict__ d_o,
                                  long long ld_do, float* __restrict__ delta,
                                  long long delta_stride, int c, int t, int b, int h, int D) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  pdl_wait();
  if (warp >= t * b * h) return;
  const int hi = warp % h;
  const int bi = (warp / h) % b;
  const int i = warp / (h * b);
  const T* po = o + (static_cast<long long>(i) * b + bi) * ld_o + hi * D;
  const T* pd = d_o + (static_cast<long long>(i) * b + bi) * ld_do + hi * D;
  float acc = 0.0f;
  for (int e = lane * 2; e < D; e += 64) {
    const float2 a = Elem<T>::unpack2(*reinterpret_cast<const uint32_t*>(po + e));
    const float2 g = Elem<T>::unpack2(*reinterpret_cast<const uint32_t*>(pd + e));
    acc += a.x * g.x + a.y * g.y;
  }
#pragma unroll
  for (int o2 = 16; o2 > 0; o2 >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o2);
  if (lane == 0) delta[static_cast<long long>(bi * h + hi) * delta_stride + c + i] = acc;
}

// ============================================================================ backward
// One streaming kernel, two modes (both deterministic, no floating-point atomics):
//   MODE 0 (dK/dV): stationary = 128 keys of the current slice (K, V tiles); streams, in
//     blocks of 64, the queries q >= k of this slice and of every later slice (Q and dO rows,
//     which later slices left in the full-length buffers).  dK/dV of a key block are therefore
//     complete when the CTA ends and are written once, as 16-bit values.
//   MODE 1 (dQ): stationary = 128 queries of the current slice (Q, dO tiles); streams the keys
//     k <= q (K, V tiles of 64 rows).
// Per streamed block:  S = X1 Y1^T, dP = X2 Y2^T (TMEM, double buffered);
//   P = exp2(S*scale2 - lse), dS = P (dP - delta)  -> 16-bit tiles in shared memory;
//   MODE 0: dV += P^T-tile * dO, dK += dS^T-tile * Q;   MODE 1: dQ += dS * K.
// 10 warps: two worker groups of 4 warps alternate over the streamed blocks (each owns one
// S/dP buffer), warp 8 elects the TMA thread, warp 9 the MMA thread.
constexpr int kBwdThreads = 320;
constexpr int kBwdMaxStages = 4;
// Ring depth of the streamed tiles: the dQ mode needs no P tile and spends that shared memory
// on a fourth stage (the streamed K/V come from HBM, so loads must run well ahead).
template <int MODE> struct BwdStages { static constexpr int value = MODE == 1 ? 4 : 3; };

struct BwdShared {
  uint64_t bar_x, bar_y[kBwdMaxStages], bar_yfree[kBwdMaxStages], bar_s[2], bar_sfree[2], bar_p[2],
      bar_acc[2], bar_done;
  alignas(16) float lse[kBwdMaxStages][64];    // MODE 0: per streamed block, bulk-copied by the producer
  alignas(16) float delta[kBwdMaxStages][64];
  uint32_t tmem_slot;
  int abort_flag;
};

template <typename T, int D, int MODE>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQKV128,
                const __grid_constant__ CUtensorMap tmQKV64,
                const __grid_constant__ CUtensorMap tmDO128,
                const __grid_constant__ CUtensorMap tmDO64, const AttnParams p) {
  constexpr int DH = D / 64;
  constexpr int kXSub = 128 * 128, kYSub = 64 * 128;
  constexpr int kStageBytes = 2 * DH * kYSub;
  constexpr int kBwdStages = BwdStages<MODE>::value;
  constexpr uint32_t kTmemCols = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sX1 = smem;
  uint8_t* sX2 = sX1 + DH * kXSub;
  uint8_t* sY = sX2 + DH * kXSub;                 // [stages][Y1 | Y2][DH][kYSub]
  uint8_t* sP = sY + kBwdStages * kStageBytes;    // [128][128B], MODE 0 only
  uint8_t* sdS = MODE == 0 ? sP + 128 * 128 : sP;
  BwdShared* sh = reinterpret_cast<BwdShared*>(sdS + 128 * 128);

  const int warp = threadIdx.x >> 5;
  const WaitCtx wctx{&sh->abort_flag, p.err};
  const int bh = blockIdx.y;
  const int bi = bh / p.h, hi = bh % p.h;
  const int x0 = p.c + blockIdx.x * 128;  // first stationary row (absolute position)
  int ystart, n_iter;
  if (MODE == 0) {
    ystart = x0;
    n_iter = (p.q_end - x0 + 63) / 64;
  } else {
    ystart = 0;
    n_iter = (p.c + min(p.t, static_cast<int>(blockIdx.x) * 128 + 128) + 63) / 64;
  }

  if (threadIdx.x == 0) {
    mbar_init(&sh->bar_x, 1);
    for (int i = 0; i < kBwdStages; ++i) {
      mbar_init(&sh->bar_y[i], 1);
      mbar_init(&sh->bar_yfree[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh->bar_s[i], 1);
      mbar_init(&sh->bar_sfree[i], 4);
      mbar_init(&sh->bar_p[i], 4);
    }
    mbar_init(&sh->bar_acc[0], 1);
    mbar_init(&sh->bar_acc[1], 1);
    mbar_init(&sh->bar_done, 1);
    sh->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 9) {
    tmem_alloc(&sh->tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();  // set-up done; from here on the predecessor's results are read
  const uint32_t tmem = sh->tmem_slot;
  // columns: S[0] 0, S[1] 64, dP[0] 128, dP[1] 192, Acc1 256, Acc2 256 + D
  const uint32_t tA1 = tmem + 256, tA2 = tmem + 256 + D;

  if (warp == 8) {
    // producer: one thread issues every bulk copy.  In MODE 0 the streamed queries' lse/delta
    // (64 contiguous floats each) ride on the same barrier as the tiles.
    if (elect_one()) {
      mbar_expect_tx(&sh->bar_x, 2 * DH * kXSub);
      for (int hh = 0; hh < DH; ++hh) {
        if (MODE == 0) {
          tma_load_3d(sX1 + hh * kXSub, &tmQKV128, &sh->bar_x, D + hh * 64, bh, x0);
          tma_load_3d(sX2 + hh * kXSub, &tmQKV128, &sh->bar_x, 2 * D + hh * 64, bh, x0);
        } else {
          tma_load_3d(sX1 + hh * kXSub, &tmQKV128, &sh->bar_x, hh * 64, bh, x0);
          tma_load_3d(sX2 + hh * kXSub, &tmDO128, &sh->bar_x, hi * D + hh * 64, bi, x0);
        }
      }
      for (int i = 0; i < n_iter; ++i) {
        const int st = i % kBwdStages;
        if (!mbar_wait(&sh->bar_yfree[st], ((i / kBwdStages) & 1) ^ 1, wctx, kErrWaitAttn)) break;
        uint8_t* y1 = sY + st * kStageBytes;
        uint8_t* y2 = y1 + DH * kYSub;
        const int y0 = ystart + i * 64;
        // a block that runs past q_end takes its lse/delta through guarded plain loads instead
        const bool bulk_stats = MODE == 0 && y0 + 64 <= p.q_end && (y0 & 3) == 0 &&
                                (p.lse_stride & 3) == 0 &&
                                TP_CHECK(y0 >= 0 && y0 + 64 <= p.lse_stride, p.err, kErrCheckAttn);
        if (MODE == 0 && !bulk_stats) {
          const long long base = static_cast<long long>(bh) * p.lse_stride;
          for (int k = 0; k < 64; ++k) {
            const bool in = y0 + k < p.q_end &&
                            TP_CHECK(y0 + k >= 0 && y0 + k < p.lse_stride, p.err, kErrCheckAttn);
            sh->lse[st][k] = in ? __ldcg(p.lse2 + base + y0 + k) : 0.0f;
            sh->delta[st][k] = in ? __ldcg(p.delta + base + y0 + k) : 0.0f;
          }
        }
        mbar_expect_tx(&sh->bar_y[st], kStageBytes + (bulk_stats ? 512 : 0));
        for (int hh = 0; hh < DH; ++hh) {
          if (MODE == 0) {
            tma_load_3d(y1 + hh * kYSub, &tmQKV64, &sh->bar_y[st], hh * 64, bh, y0);
            tma_load_3d(y2 + hh * kYSub, &tmDO64, &sh->bar_y[st], hi * D + hh * 64, bi, y0);
          } else {
            tma_load_3d(y1 + hh * kYSub, &tmQKV64, &sh->bar_y[st], D + hh * 64, bh, y0);
            tma_load_3d(y2 + hh * kYSub, &tmQKV64, &sh->bar_y[st], 2 * D + hh * 64, bh, y0);
          }
        }
        if (bulk_stats) {
          const long long off = static_cast<long long>(bh) * p.lse_stride + y0;
          bulk_load_1d(sh->lse[st], p.lse2 + off, 256, &sh->bar_y[st]);
          bulk_load_1d(sh->delta[st], p.delta + off, 256, &sh->bar_y[st]);
        }
      }
    }
  } else if (warp == 9) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = umma_idesc_f16(Elem<T>::fmt, 0, 0, 128, 64);
      constexpr uint32_t idesc_g = umma_idesc_f16(Elem<T>::fmt, 0, 1, 128, D);
      bool ok = mbar_wait(&sh->bar_x, 0, wctx, kErrWaitAttn);
      auto issue_acc = [&](int j) -> bool {
        if (!mbar_wait(&sh->bar_p[j & 1], (j >> 1) & 1, wctx, kErrWaitAttn)) return false;
        tc_fence_after();
        const int st = j % kBwdStages;
        const uint32_t y1 = smem_u32(sY + st * kStageBytes);
        const uint32_t y2 = y1 + DH * kYSub;
        if (MODE == 0) mma_kn(tA1, smem_u32(sP), y2, kYSub, idesc_g, j > 0);
        mma_kn(tA2, smem_u32(sdS), y1, kYSub, idesc_g, j > 0);
        umma_commit(&sh->bar_yfree[st]);
        umma_commit(&sh->bar_acc[j & 1]);
        return true;
      };
      for (int i = 0; i < n_iter && ok; ++i) {
        const int st = i % kBwdStages, buf = i & 1;
        ok = mbar_wait(&sh->bar_y[st], (i / kBwdStages) & 1, wctx, kErrWaitAttn) &&
             mbar_wait(&sh->bar_sfree[buf], ((i >> 1) & 1) ^ 1, wctx, kErrWaitAttn);
        if (!ok) break;
        tc_fence_after();
        const uint32_t y1 = smem_u32(sY + st * kStageBytes);
        const uint32_t y2 = y1 + DH * kYSub;
        mma_kk<DH>(tmem + buf * 64, smem_u32(sX1), kXSub, y1, kYSub, idesc_s);
        mma_kk<DH>(tmem + 128 + buf * 64, smem_u32(sX2), kXSub, y2, kYSub, idesc_s);
        umma_commit(&sh->bar_s[buf]);
        if (i >= 1) ok = issue_acc(i - 1);
      }
      if (ok && n_iter > 0) ok = issue_acc(n_iter - 1);
      if (ok) umma_commit(&sh->bar_done);
    }
  } else {
    const int grp = warp >> 2;                 // worker group 0 / 1
    const int r = threadIdx.x & 127;           // row of the stationary tile = TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int xabs = x0 + r;                   // absolute position of this thread's row
    // checked build: the row's statistics slot and its columns of the gradient exist
    const bool x_ok = xabs < p.c + p.t &&
                      TP_CHECK(xabs >= p.c && xabs < p.lse_stride && (hi + 1) * 3 * D <= p.ld_dqkv, p.err,
                               kErrCheckAttn);
    float lse_r = 0.0f, delta_r = 0.0f;
    if (MODE == 1 && x_ok) {
      lse_r = p.lse2[static_cast<long long>(bh) * p.lse_stride + xabs];
      delta_r = p.delta[static_cast<long long>(bh) * p.lse_stride + xabs];
    }
    bool ok = true;
    for (int i = grp; i < n_iter; i += 2) {
      const int y0 = ystart + i * 64;
      const int st = i % kBwdStages;
      ok = mbar_wait(&sh->bar_s[grp], (i >> 1) & 1, wctx, kErrWaitAttn);
      if (!ok) break;
      tc_fence_after();
      float sv[64], dv[64];
      {
        uint32_t r0[32], r1[32], r2[32], r3[32];
        __syncwarp();
        tmem_ld_32x32(tmem + grp * 64 + lane_base, r0);
        tmem_ld_32x32(tmem + grp * 64 + lane_base + 32, r1);
        tmem_ld_32x32(tmem + 128 + grp * 64 + lane_base, r2);
        tmem_ld_32x32(tmem + 128 + grp * 64 + lane_base + 32, r3);
        tmem_ld_wait();
#pragma unroll
        for (int k = 0; k < 32; ++k) {
          sv[k] = __uint_as_float(r0[k]);
          sv[32 + k] = __uint_as_float(r1[k]);
          dv[k] = __uint_as_float(r2[k]);
          dv[32 + k] = __uint_as_float(r3[k]);
        }
      }
      tc_fence_before();
      warp_arrive(&sh->bar_sfree[grp]);
      // blocks strictly inside the causal region need no per-element mask
      const bool full = MODE == 0 ? (y0 >= x0 + 127 && y0 + 64 <= p.q_end) : (y0 + 63 <= x0);
      if (full) {
#pragma unroll
        for (int k = 0; k < 64; ++k) {
          const float l2 = MODE == 0 ? sh->lse[st][k] : lse_r;
          const float dl = MODE == 0 ? sh->delta[st][k] : delta_r;
          const float pr = exp2f(sv[k] * p.scale2 - l2);
          dv[k] = pr * (dv[k] - dl);
          sv[k] = pr;
        }
      } else {
#pragma unroll
        for (int k = 0; k < 64; ++k) {
          const int yabs = y0 + k;
          const float l2 = MODE == 0 ? sh->lse[st][k] : lse_r;
          const float dl = MODE == 0 ? sh->delta[st][k] : delta_r;
          const bool valid = MODE == 0 ? ((yabs < p.q_end) && (xabs <= yabs)) : (x_ok && (yabs <= xabs));
          const float pr = valid ? exp2f(sv[k] * p.scale2 - l2) : 0.0f;
          dv[k] = pr * (dv[k] - dl);
          sv[k] = pr;
        }
      }
      // the operand tiles are free once the accumulating MMAs of the previous block are done
      if (i >= 1) ok = mbar_wait(&sh->bar_acc[(i - 1) & 1], ((i - 1) >> 1) & 1, wctx, kErrWaitAttn);
      if (!ok) break;
      if (MODE == 0) store_row64<T>(sP, r, sv);
      store_row64<T>(sdS, r, dv);
      fence_proxy_async();
      tc_fence_before();
      warp_arrive(&sh->bar_p[grp]);
    }
    if (ok && n_iter > 0) ok = mbar_wait(&sh->bar_done, 0, wctx, kErrWaitAttn);
    if (ok && n_iter > 0) {
      tc_fence_after();
      const long long out_row = (static_cast<long long>(xabs - p.c) * p.b + bi) * p.ld_dqkv + hi * 3 * D;
      T* drow = static_cast<T*>(p.dqkv) + out_row;
      uint32_t tsrc;
      int col0, ncols, slot;
      float mul;
      if (MODE == 0) {   // group 0: dV (Acc1) -> v slot; group 1: dK (Acc2) * scale -> k slot
        tsrc = grp == 0 ? tA1 : tA2;
        col0 = 0; ncols = D; slot = grp == 0 ? 2 * D : D;
        mul = grp == 0 ? 1.0f : p.scale;
      } else {           // dQ (Acc2) * scale -> q slot, each group writes half of the columns
        tsrc = tA2;
        col0 = grp * (D / 2); ncols = D / 2; slot = 0;
        mul = p.scale;
      }
#pragma unroll 1
      for (int cc = col0; cc < col0 + ncols; cc += 32) {
        uint32_t raw[32];
        __syncwarp();
        tmem_ld_32x32(tsrc + lane_base + cc, raw);
        tmem_ld_wait();
        if (x_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 u;
            u.x = Elem<T>::pack2(__uint_as_float(raw[g * 8 + 0]) * mul, __uint_as_float(raw[g * 8 + 1]) * mul);
            u.y = Elem<T>::pack2(__uint_as_float(raw[g * 8 + 2]) * mul, __uint_as_float(raw[g * 8 + 3]) * mul);
            u.z = Elem<T>::pack2(__uint_as_float(raw[g * 8 + 4]) * mul, __uint_as_float(raw[g * 8 + 5]) * mul);
            u.w = Elem<T>::pack2(__uint_as_float(raw[g * 8 + 6]) * mul, __uint_as_float(raw[g * 8 + 7]) * mul);
            __stcg(reinterpret_cast<uint4*>(drow + slot + cc + g * 8), u);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (sh->abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_after();
  if (warp == 9) tmem_dealloc(tmem, kTmemCols);
}

// ---------------------------------------------------------------------------- host side
static bool qkv_tmap(CUtensorMap* out, const void* qkv, int D, int b, int h, int rows_valid,
                     int box_rows, bool bf16) {
  uint64_t dims[3] = {static_cast<uint64_t>(3 * D), static_cast<uint64_t>(b * h),
                      static_cast<uint64_t>(rows_valid)};
  uint64_t strides[2] = {static_cast<uint64_t>(3 * D) * 2, static_cast<uint64_t>(b) * h * 3 * D * 2};
  uint32_t box[3] = {64, 1, static_cast<uint32_t>(box_rows)};
  return make_tmap_16b(out, qkv, 3, dims, strides, box, bf16);
}

static bool do_tmap(CUtensorMap* out, const void* d_o, long long ld, int D, int b, int h, int t,
                    int box_rows, bool bf16) {
  uint64_t dims[3] = {static_cast<uint64_t>(h * D), static_cast<uint64_t>(b), static_cast<uint64_t>(t)};
  uint64_t strides[2] = {static_cast<uint64_t>(ld) * 2, static_cast<uint64_t>(b) * ld * 2};
  uint32_t box[3] = {64, 1, static_cast<uint32_t>(box_rows)};
  return make_tmap_16b(out, d_o, 3, dims, strides, box, bf16);
}

template <typename K> static bool set_smem(K kern, int bytes) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess;
}

template <int D> constexpr int fwd_smem() { return (D / 64) * (128 * 128 + 8 * 64 * 128) + 2 * 128 * 128 + 1024 + 512; }
template <int D, int MODE> constexpr int bwd_smem() {
  return (D / 64) * (2 * 128 * 128 + BwdStages<MODE>::value * 2 * 64 * 128) +
         (MODE == 0 ? 2 : 1) * 128 * 128 + 1024 +
         static_cast<int>(sizeof(BwdShared)) + 64;
}

template <typename T, int D>
static int attn_fwd_launch(const void* qkv, const AttnParams& p, bool bf16, cudaStream_t s) {
  CUtensorMap tmQ, tmKV;
  if (!qkv_tmap(&tmQ, qkv, D, p.b, p.h, p.c + p.t, 128, bf16) ||
      !qkv_tmap(&tmKV, qkv, D, p.b, p.h, p.c + p.t, 64, bf16))
    return kErrDriver;
  auto kern = attn_fwd_kernel<T, D>;
  static bool cfg = false;
  if (!cfg) { if (!set_smem(kern, fwd_smem<D>())) return kErrLaunch; cfg = true; }
  dim3 grid((p.t + 127) / 128, p.b * p.h);
  return launch_pdl(kern, grid, dim3(kAttnThreads), fwd_smem<D>(), s, 1, tmQ, tmKV, p) == cudaSuccess
             ? kOk
             : kErrLaunch;
}

template <typename T, int D>
static int attn_bwd_launch(const void* qkv, const void* o, const void* do_full, long long ld_do,
                           const AttnParams& p, bool bf16, cudaStream_t s) {
  CUtensorMap tm128, tm64, tmdO64, tmdO128;
  if (!qkv_tmap(&tm128, qkv, D, p.b, p.h, p.q_end, 128, bf16) ||
      !qkv_tmap(&tm64, qkv, D, p.b, p.h, p.q_end, 64, bf16) ||
      !do_tmap(&tmdO64, do_full, ld_do, D, p.b, p.h, p.q_end, 64, bf16) ||
      !do_tmap(&tmdO128, do_full, ld_do, D, p.b, p.h, p.q_end, 128, bf16))
    return kErrDriver;
  {
    const long long warps = static_cast<long long>(p.t) * p.b * p.h;
    const int threads = 256;
    const int blocks = static_cast<int>((warps * 32 + threads - 1) / threads);
    const T* do_slice = static_cast<const T*>(do_full) + static_cast<long long>(p.c) * p.b * ld_do;
    if (launch_pdl(attn_delta_kernel<T>, dim3(blocks), dim3(threads), 0, s, 1, static_cast<const T*>(o),
                   p.ld_o, do_slice, ld_do, p.delta, p.lse_stride, p.c, p.t, p.b, p.h, D) != cudaSuccess)
      return kErrLaunch;
  }
  auto k0 = attn_bwd_kernel<T, D, 0>;
  auto k1 = attn_bwd_kernel<T, D, 1>;
  static bool cfg = false;
  if (!cfg) {
    if (!set_smem(k0, bwd_smem<D, 0>()) || !set_smem(k1, bwd_smem<D, 1>())) return kErrLaunch;
    cfg = true;
  }
  dim3 grid((p.t + 127) / 128, p.b * p.h);
  if (launch_pdl(k0, grid, dim3(kBwdThreads), bwd_smem<D, 0>(), s, 1, tm128, tm64, tmdO128, tmdO64, p) !=
      cudaSuccess)
    return kErrLaunch;
  return launch_pdl(k1, grid, dim3(kBwdThreads), bwd_smem<D, 1>(), s, 1, tm128, tm64, tmdO128, tmdO64, p) ==
                 cudaSuccess
             ? kOk
             : kErrLaunch;
}

}  // namespace tp

using namespace tp;

// `scale` multiplies q.k before the softmax; <= 0 selects D^-0.5.  A caller whose heads are narrower
// than the kernel's D (zero-padded columns) passes the scale of the real width.
static AttnParams base_params(int D, float scale, int b, int h, int t, int c, int* err) {
  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.t = t; p.c = c; p.b = b; p.h = h;
  p.scale = scale > 0.0f ? scale : 1.0f / sqrtf(static_cast<float>(D));
  p.scale2 = p.scale * 1.4426950408889634f;
  p.err = err;
  return p;
}

// qkv: base of the full-length [L][b][h][3][D] buffer; rows [0, c+t) must be valid.
extern "C" int tp_attn_fwd_scaled(int dtype, int D, float scale, const void* qkv, int b, int h, int t,
                                  int c, void* o, long long ld_o, float* lse2, long long lse_stride,
                                  int* err, void* stream) {
  if ((D != 64 && D != 128) || t <= 0 || c < 0 || b <= 0 || h <= 0) return kErrBadArgument;
  if (ld_o % 8) return kErrBadArgument;
  AttnParams p = base_params(D, scale, b, h, t, c, err);
  p.o = o; p.ld_o = ld_o; p.lse2 = lse2; p.lse_stride = lse_stride;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool bf16 = dtype == 1;
  if (D == 128) return bf16 ? attn_fwd_launch<__nv_bfloat16, 128>(qkv, p, true, s)
                            : attn_fwd_launch<__half, 128>(qkv, p, false, s);
  return bf16 ? attn_fwd_launch<__nv_bfloat16, 64>(qkv, p, true, s)
              : attn_fwd_launch<__half, 64>(qkv, p, false, s);
}

extern "C" int tp_attn_fwd(int dtype, int D, const void* qkv, int b, int h, int t, int c, void* o,
                           long long ld_o, float* lse2, long long lse_stride, int* err,
                           void* stream) {
  return tp_attn_fwd_scaled(dtype, D, 0.0f, qkv, b, h, t, c, o, ld_o, lse2, lse_stride, err, stream);
}

// Backward of the slice [c, c+t).  The slices after it must already have been processed:
//   o        this slice's attention output, [t*b][ld_o]
//   do_full  full-length gradient of the attention output, [L*b][ld_do]; rows [c*b, q_end*b)
//            are read (this slice's rows must have been written by the caller)
//   lse2, delta   fp32 [b*h][lse_stride], indexed by absolute position; delta rows [c, c+t) are
//            written here, rows [c+t, q_end) were written by the calls for the later slices
//   dqkv     this slice's [t*b][ld_dqkv] output (same column order as qkv)
extern "C" int tp_attn_bwd_scaled(int dtype, int D, float scale, const void* qkv, int b, int h, int t,
                                  int c, int q_end, const void* o, long long ld_o, const void* do_full,
                                  long long ld_do, const float* lse2, long long lse_stride,
                                  float* delta, void* dqkv, long long ld_dqkv, int* err,
                                  void* stream) {
  if ((D != 64 && D != 128) || t <= 0 || c < 0 || b <= 0 || h <= 0 || q_end < c + t)
    return kErrBadArgument;
  if (ld_o % 8 || ld_do % 8 || ld_dqkv % 8) return kErrBadArgument;
  AttnParams p = base_params(D, scale, b, h, t, c, err);
  p.o = const_cast<void*>(o); p.ld_o = ld_o;
  p.lse2 = const_cast<float*>(lse2); p.lse_stride = lse_stride;
  p.delta = delta; p.q_end = q_end; p.dqkv = dqkv; p.ld_dqkv = ld_dqkv;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool bf16 = dtype == 1;
  if (D == 128) return bf16 ? attn_bwd_launch<__nv_bfloat16, 128>(qkv, o, do_full, ld_do, p, true, s)
                            : attn_bwd_launch<__half, 128>(qkv, o, do_full, ld_do, p, false, s);
  return bf16 ? attn_bwd_launch<__nv_bfloat16, 64>(qkv, o, do_full, ld_do, p, true, s)
              : attn_bwd_launch<__half, 64>(qkv, o, do_full, ld_do, p, false, s);
}

extern "C" int tp_attn_bwd(int dtype, int D, const void* qkv, int b, int h, int t, int c, int q_end,
                           const void* o, long long ld_o, const void* do_full, long long ld_do,
                           const float* lse2, long long lse_stride, float* delta, void* dqkv,
                           long long ld_dqkv, int* err, void* stream) {
  return tp_attn_bwd_scaled(dtype, D, 0.0f, qkv, b, h, t, c, q_end, o, ld_o, do_full, ld_do, lse2,
                            lse_stride, delta, dqkv, ld_dqkv, err, stream);
}

TP_DEFINE_WAIT_LIMIT_SETTER(tp_set_wait_limit_ns_attn)
