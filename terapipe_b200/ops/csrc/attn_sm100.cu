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
// Backward recomputes P from Q, K and the saved log-sum-exp (base 2).  Two kernels, both
// deterministic (no floating-point atomics):
//   * dK/dV: one CTA per (128-key block, head); loops over the slice's query blocks and adds
//     its result into a persistent fp32 accumulator dkv[b][h][L][2][D] that lives across the
//     slices of one backward pass; rows of the current slice are final and are also written
//     as 16-bit values into the slice's d(qkv) buffer for the QKV weight/data gradients.
//   * dQ:    one CTA per (128-query block, head); loops over key blocks.
//
// CTA = 5 warps: warps 0..3 own one TMEM lane quarter each (one row per thread: softmax needs
// no shuffles), warp 4 elects one thread that issues all TMA copies and MMAs.
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
  const float* delta;   // bwd: [b*h][t] = rowsum(dO * O)
  float* dkv_acc;       // [b*h][dkv_rows][2][D] fp32 (head-major: a CTA's key rows are contiguous)
  long long dkv_rows;
  void* dqkv;           // [t*b][ld_dqkv], same column order as qkv
  long long ld_dqkv;
  int first;            // dK/dV: overwrite the accumulator instead of adding to it
  int* err;
};

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
  uint64_t bars[12];
  uint32_t tmem_slot;
  int abort_flag;
};

// ============================================================================ forward
template <typename T, int D>
__global__ void __launch_bounds__(kAttnThreads, D == 128 ? 2 : 3)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV,
                const AttnParams p) {
  constexpr int DH = D / 64;
  constexpr int kQSub = 128 * 128, kKSub = 64 * 128;
  constexpr uint32_t kTmemCols = D == 128 ? 256 : 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + DH * kQSub;
  uint8_t* sV = sK + DH * kKSub;
  uint8_t* sP = sV + DH * kKSub;
  AttnShared* sh = reinterpret_cast<AttnShared*>(sP + 128 * 128);
  uint64_t* bar_q = &sh->bars[0];
  uint64_t* bar_k = &sh->bars[1];
  uint64_t* bar_v = &sh->bars[2];
  uint64_t* bar_s = &sh->bars[3];
  uint64_t* bar_p = &sh->bars[4];
  uint64_t* bar_pv = &sh->bars[5];

  const int warp = threadIdx.x >> 5;
  const WaitCtx wctx{&sh->abort_flag, p.err};
  const int q0 = blockIdx.x * 128;
  const int bh = blockIdx.y;
  const int bi = bh / p.h, hi = bh % p.h;
  const int q_hi = min(p.t, q0 + 128);
  const int nkb = (p.c + q_hi + 63) / 64;

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_k, 1);
    mbar_init(bar_v, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_p, 128);
    mbar_init(bar_pv, 1);
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
  const uint32_t tmem = sh->tmem_slot;
  const uint32_t tS = tmem, tO = tmem + 64;

  if (warp == 4) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = umma_idesc_f16(Elem<T>::fmt, 0, 0, 128, 64);
      constexpr uint32_t idesc_pv = umma_idesc_f16(Elem<T>::fmt, 0, 1, 128, D);
      mbar_expect_tx(bar_q, DH * kQSub);
      for (int hh = 0; hh < DH; ++hh)
        tma_load_3d(sQ + hh * kQSub, &tmQ, bar_q, hh * 64, bh, p.c + q0);
      mbar_expect_tx(bar_k, DH * kKSub);
      for (int hh = 0; hh < DH; ++hh) tma_load_3d(sK + hh * kKSub, &tmKV, bar_k, D + hh * 64, bh, 0);
      mbar_expect_tx(bar_v, DH * kKSub);
      for (int hh = 0; hh < DH; ++hh)
        tma_load_3d(sV + hh * kKSub, &tmKV, bar_v, 2 * D + hh * 64, bh, 0);
      bool ok = mbar_wait(bar_q, 0, wctx, kErrWaitAttn);
      for (int j = 0; j < nkb && ok; ++j) {
        const uint32_t ph = j & 1;
        ok = mbar_wait(bar_k, ph, wctx, kErrWaitAttn);
        if (!ok) break;
        tc_fence_after();
        mma_kk<DH>(tS, smem_u32(sQ), kQSub, smem_u32(sK), kKSub, idesc_s);
        umma_commit(bar_s);
        ok = mbar_wait(bar_s, ph, wctx, kErrWaitAttn);
        if (!ok) break;
        if (j + 1 < nkb) {
          mbar_expect_tx(bar_k, DH * kKSub);
          for (int hh = 0; hh < DH; ++hh)
            tma_load_3d(sK + hh * kKSub, &tmKV, bar_k, D + hh * 64, bh, (j + 1) * 64);
        }
        ok = mbar_wait(bar_p, ph, wctx, kErrWaitAttn) && mbar_wait(bar_v, ph, wctx, kErrWaitAttn);
        if (!ok) break;
        tc_fence_after();
        mma_kn(tO, smem_u32(sP), smem_u32(sV), kKSub, idesc_pv, j > 0);
        umma_commit(bar_pv);
        ok = mbar_wait(bar_pv, ph, wctx, kErrWaitAttn);
        if (!ok) break;
        if (j + 1 < nkb) {
          mbar_expect_tx(bar_v, DH * kKSub);
          for (int hh = 0; hh < DH; ++hh)
            tma_load_3d(sV + hh * kKSub, &tmKV, bar_v, 2 * D + hh * 64, bh, (j + 1) * 64);
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
      ok = mbar_wait(bar_s, j & 1, wctx, kErrWaitAttn);
      if (!ok) break;
      tc_fence_after();
      float s[64];
      {
        uint32_t raw[32];
        __syncwarp();
        tmem_ld_32x32(tS + lane_base, raw);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) s[i] = __uint_as_float(raw[i]);
        tmem_ld_32x32(tS + lane_base + 32, raw);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) s[32 + i] = __uint_as_float(raw[i]);
      }
      float mx = -INFINITY;
      const int kbase = j * 64;
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        s[i] = (kbase + i <= qpos) ? s[i] * p.scale2 : -INFINITY;
        mx = fmaxf(mx, s[i]);
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
      store_row64<T>(sP, r, s);
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(bar_p);
    }
    if (ok) ok = mbar_wait(bar_pv, (nkb - 1) & 1, wctx, kErrWaitAttn);
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.0f / l;
      T* orow = static_cast<T*>(p.o) + (static_cast<long long>(qi) * p.b + bi) * p.ld_o + hi * D;
#pragma unroll 1
      for (int ch = 0; ch < D / 32; ++ch) {
        uint32_t raw[32];
        __syncwarp();
        tmem_ld_32x32(tO + lane_base + ch * 32, raw);
        tmem_ld_wait();
        if (qi < p.t) {
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
      if (qi < p.t) p.lse2[static_cast<long long>(bh) * p.lse_stride + qpos] = m + log2f(l);
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
                                  long long ld_do, float* __restrict__ delta, int t, int b, int h,
                                  int D) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
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
  if (lane == 0) delta[static_cast<long long>(bi * h + hi) * t + i] = acc;
}

// ============================================================================ backward: dK, dV
template <typename T, int D>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmKV128,
                     const __grid_constant__ CUtensorMap tmQ64,
                     const __grid_constant__ CUtensorMap tmdO64, const AttnParams p) {
  constexpr int DH = D / 64;
  constexpr int kKSub = 128 * 128, kQSub = 64 * 128;
  constexpr uint32_t kTmemCols = D == 128 ? 512 : 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + DH * kKSub;
  uint8_t* sQ = sV + DH * kKSub;         // [2][DH][kQSub]
  uint8_t* sdO = sQ + 2 * DH * kQSub;    // [2][DH][kQSub]
  uint8_t* sPt = sdO + 2 * DH * kQSub;   // [128][128B]
  uint8_t* sdSt = sPt + 128 * 128;
  float* s_lse = reinterpret_cast<float*>(sdSt + 128 * 128);  // [2][64]
  float* s_delta = s_lse + 128;                               // [2][64]
  AttnShared* sh = reinterpret_cast<AttnShared*>(s_delta + 128);
  uint64_t* bar_kv = &sh->bars[0];
  uint64_t* bar_qdo = &sh->bars[1];  // [2]
  uint64_t* bar_s = &sh->bars[3];
  uint64_t* bar_p = &sh->bars[4];
  uint64_t* bar_m2 = &sh->bars[5];

  const int warp = threadIdx.x >> 5;
  const WaitCtx wctx{&sh->abort_flag, p.err};
  const int k0 = blockIdx.x * 128;
  const int bh = blockIdx.y;
  const int bi = bh / p.h, hi = bh % p.h;
  const int qb_start = (k0 > p.c ? (k0 - p.c) : 0) / 64;
  const int nqb = (p.t + 63) / 64;
  const int nit = nqb - qb_start;

  if (threadIdx.x == 0) {
    mbar_init(bar_kv, 1);
    mbar_init(&bar_qdo[0], 1);
    mbar_init(&bar_qdo[1], 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_p, 128);
    mbar_init(bar_m2, 1);
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
  const uint32_t tmem = sh->tmem_slot;
  const uint32_t tSt = tmem, tdPt = tmem + 64, tdV = tmem + 128, tdK = tmem + 128 + D;

  if (warp == 4) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = umma_idesc_f16(Elem<T>::fmt, 0, 0, 128, 64);
      constexpr uint32_t idesc_g = umma_idesc_f16(Elem<T>::fmt, 0, 1, 128, D);
      mbar_expect_tx(bar_kv, 2 * DH * kKSub);
      for (int hh = 0; hh < DH; ++hh) {
        tma_load_3d(sK + hh * kKSub, &tmKV128, bar_kv, D + hh * 64, bh, k0);
        tma_load_3d(sV + hh * kKSub, &tmKV128, bar_kv, 2 * D + hh * 64, bh, k0);
      }
      auto load_q = [&](int qb, int st) {
        mbar_expect_tx(&bar_qdo[st], 2 * DH * kQSub);
        for (int hh = 0; hh < DH; ++hh) {
          tma_load_3d(sQ + (st * DH + hh) * kQSub, &tmQ64, &bar_qdo[st], hh * 64, bh,
                      p.c + qb * 64);
          tma_load_3d(sdO + (st * DH + hh) * kQSub, &tmdO64, &bar_qdo[st], hi * D + hh * 64, bi,
                      qb * 64);
        }
      };
      load_q(qb_start, 0);
      bool ok = mbar_wait(bar_kv, 0, wctx, kErrWaitAttn);
      for (int it = 0; it < nit && ok; ++it) {
        const int st = it & 1;
        if (it + 1 < nit) load_q(qb_start + it + 1, st ^ 1);
        ok = mbar_wait(&bar_qdo[st], (it >> 1) & 1, wctx, kErrWaitAttn);
        if (!ok) break;
        tc_fence_after();
        const uint32_t q_base = smem_u32(sQ + st * DH * kQSub);
        const uint32_t do_base = smem_u32(sdO + st * DH * kQSub);
        mma_kk<DH>(tSt, smem_u32(sK), kKSub, q_base, kQSub, idesc_s);
        mma_kk<DH>(tdPt, smem_u32(sV), kKSub, do_base, kQSub, idesc_s);
        umma_commit(bar_s);
        ok = mbar_wait(bar_p, it & 1, wctx, kErrWaitAttn);
        if (!ok) break;
        tc_fence_after();
        mma_kn(tdV, smem_u32(sPt), do_base, kQSub, idesc_g, it > 0);
        mma_kn(tdK, smem_u32(sdSt), q_base, kQSub, idesc_g, it > 0);
        umma_commit(bar_m2);
        ok = mbar_wait(bar_m2, it & 1, wctx, kErrWaitAttn);
      }
    }
  } else {
    const int r = threadIdx.x;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const int kpos = k0 + r;
    bool ok = true;
    for (int it = 0; it < nit; ++it) {
      const int st = it & 1;
      const int qb = qb_start + it;
      {
        const int qi = qb * 64 + (r & 63);
        if (r < 64)
          s_lse[st * 64 + r] = qi < p.t ? p.lse2[static_cast<long long>(bh) * p.lse_stride + p.c + qi] : 0.0f;
        else
          s_delta[st * 64 + (r - 64)] = qi < p.t ? p.delta[static_cast<long long>(bh) * p.t + qi] : 0.0f;
      }
      named_bar_sync(1, 128);  // every worker reaches this in every iteration, aborted or not
      if (ok) ok = mbar_wait(bar_s, it & 1, wctx, kErrWaitAttn);
      if (!ok) continue;
      tc_fence_after();
      float sv[64], dv[64];
      {
        uint32_t raw[32];
        __syncwarp();
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          tmem_ld_32x32(tSt + lane_base + half * 32, raw);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) sv[half * 32 + i] = __uint_as_float(raw[i]);
          tmem_ld_32x32(tdPt + lane_base + half * 32, raw);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) dv[half * 32 + i] = __uint_as_float(raw[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        const int qi = qb * 64 + i;
        const bool valid = (qi < p.t) && (kpos <= p.c + qi);
        const float pr = valid ? exp2f(sv[i] * p.scale2 - s_lse[st * 64 + i]) : 0.0f;
        sv[i] = pr;
        dv[i] = pr * (dv[i] - s_delta[st * 64 + i]);
      }
      store_row64<T>(sPt, r, sv);
      store_row64<T>(sdSt, r, dv);
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(bar_p);
    }
    if (ok && nit > 0) ok = mbar_wait(bar_m2, (nit - 1) & 1, wctx, kErrWaitAttn);
    if (ok && nit > 0) {
      tc_fence_after();
      const bool row_ok = kpos < p.c + p.t;
      const bool final_row = kpos >= p.c;
      float* acc = p.dkv_acc + (static_cast<long long>(bh) * p.dkv_rows + kpos) * 2 * D;
      T* drow = static_cast<T*>(p.dqkv) +
                (static_cast<long long>(kpos - p.c) * p.b + bi) * p.ld_dqkv + hi * 3 * D;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {  // 0: dK (scaled), 1: dV
        const uint32_t tsrc = which == 0 ? tdK : tdV;
        const float mul = which == 0 ? p.scale : 1.0f;
#pragma unroll 1
        for (int ch = 0; ch < D / 32; ++ch) {
          uint32_t raw[32];
          __syncwarp();
          tmem_ld_32x32(tsrc + lane_base + ch * 32, raw);
          tmem_ld_wait();
          if (!row_ok) continue;
          float* a = acc + which * D + ch * 32;
          float4 oldv[8];
          if (!p.first) {
#pragma unroll
            for (int g = 0; g < 8; ++g) oldv[g] = __ldcg(reinterpret_cast<const float4*>(a + g * 4));
          }
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            float4 v = make_float4(__uint_as_float(raw[g * 4 + 0]) * mul, __uint_as_float(raw[g * 4 + 1]) * mul,
                                   __uint_as_float(raw[g * 4 + 2]) * mul, __uint_as_float(raw[g * 4 + 3]) * mul);
            if (!p.first) {
              v.x += oldv[g].x; v.y += oldv[g].y; v.z += oldv[g].z; v.w += oldv[g].w;
            }
            if (final_row) {
              uint2 u;
              u.x = Elem<T>::pack2(v.x, v.y);
              u.y = Elem<T>::pack2(v.z, v.w);
              *reinterpret_cast<uint2*>(drow + (1 + which) * D + ch * 32 + g * 4) = u;
            } else {
              __stcg(reinterpret_cast<float4*>(a + g * 4), v);
            }
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
  if (warp == 4) tmem_dealloc(tmem, kTmemCols);
}

// ============================================================================ backward: dQ
template <typename T, int D>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ128,
                   const __grid_constant__ CUtensorMap tmKV64,
                   const __grid_constant__ CUtensorMap tmdO128, const AttnParams p) {
  constexpr int DH = D / 64;
  constexpr int kQSub = 128 * 128, kKSub = 64 * 128;
  constexpr uint32_t kTmemCols = D == 128 ? 256 : 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + DH * kQSub;
  uint8_t* sK = sdO + DH * kQSub;       // [2][DH][kKSub]
  uint8_t* sV = sK + 2 * DH * kKSub;    // [2][DH][kKSub]
  uint8_t* sdS = sV + 2 * DH * kKSub;   // [128][128B]
  AttnShared* sh = reinterpret_cast<AttnShared*>(sdS + 128 * 128);
  uint64_t* bar_q = &sh->bars[0];
  uint64_t* bar_kv = &sh->bars[1];  // [2]
  uint64_t* bar_s = &sh->bars[3];
  uint64_t* bar_p = &sh->bars[4];
  uint64_t* bar_m2 = &sh->bars[5];

  const int warp = threadIdx.x >> 5;
  const WaitCtx wctx{&sh->abort_flag, p.err};
  const int q0 = blockIdx.x * 128;
  const int bh = blockIdx.y;
  const int bi = bh / p.h, hi = bh % p.h;
  const int q_hi = min(p.t, q0 + 128);
  const int nkb = (p.c + q_hi + 63) / 64;

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    mbar_init(&bar_kv[0], 1);
    mbar_init(&bar_kv[1], 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_p, 128);
    mbar_init(bar_m2, 1);
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
  const uint32_t tmem = sh->tmem_slot;
  const uint32_t tS = tmem, tdP = tmem + 64, tdQ = tmem + 128;

  if (warp == 4) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = umma_idesc_f16(Elem<T>::fmt, 0, 0, 128, 64);
      constexpr uint32_t idesc_g = umma_idesc_f16(Elem<T>::fmt, 0, 1, 128, D);
      mbar_expect_tx(bar_q, 2 * DH * kQSub);
      for (int hh = 0; hh < DH; ++hh) {
        tma_load_3d(sQ + hh * kQSub, &tmQ128, bar_q, hh * 64, bh, p.c + q0);
        tma_load_3d(sdO + hh * kQSub, &tmdO128, bar_q, hi * D + hh * 64, bi, q0);
      }
      auto load_kv = [&](int j, int st) {
        mbar_expect_tx(&bar_kv[st], 2 * DH * kKSub);
        for (int hh = 0; hh < DH; ++hh) {
          tma_load_3d(sK + (st * DH + hh) * kKSub, &tmKV64, &bar_kv[st], D + hh * 64, bh, j * 64);
          tma_load_3d(sV + (st * DH + hh) * kKSub, &tmKV64, &bar_kv[st], 2 * D + hh * 64, bh, j * 64);
        }
      };
      load_kv(0, 0);
      bool ok = mbar_wait(bar_q, 0, wctx, kErrWaitAttn);
      for (int j = 0; j < nkb && ok; ++j) {
        const int st = j & 1;
        if (j + 1 < nkb) load_kv(j + 1, st ^ 1);
        ok = mbar_wait(&bar_kv[st], (j >> 1) & 1, wctx, kErrWaitAttn);
        if (!ok) break;
        tc_fence_after();
        const uint32_t k_base = smem_u32(sK + st * DH * kKSub);
        const uint32_t v_base = smem_u32(sV + st * DH * kKSub);
        mma_kk<DH>(tS, smem_u32(sQ), kQSub, k_base, kKSub, idesc_s);
        mma_kk<DH>(tdP, smem_u32(sdO), kQSub, v_base, kKSub, idesc_s);
        umma_commit(bar_s);
        ok = mbar_wait(bar_p, j & 1, wctx, kErrWaitAttn);
        if (!ok) break;
        tc_fence_after();
        mma_kn(tdQ, smem_u32(sdS), k_base, kKSub, idesc_g, j > 0);
        umma_commit(bar_m2);
        ok = mbar_wait(bar_m2, j & 1, wctx, kErrWaitAttn);
      }
    }
  } else {
    const int r = threadIdx.x;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const int qi = q0 + r;
    const int qpos = p.c + qi;
    const bool q_ok = qi < p.t;
    const float lse_r = q_ok ? p.lse2[static_cast<long long>(bh) * p.lse_stride + qpos] : 0.0f;
    const float delta_r = q_ok ? p.delta[static_cast<long long>(bh) * p.t + qi] : 0.0f;
    bool ok = true;
    for (int j = 0; j < nkb; ++j) {
      ok = mbar_wait(bar_s, j & 1, wctx, kErrWaitAttn);
      if (!ok) break;
      tc_fence_after();
      float sv[64], dv[64];
      {
        uint32_t raw[32];
        __syncwarp();
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          tmem_ld_32x32(tS + lane_base + half * 32, raw);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) sv[half * 32 + i] = __uint_as_float(raw[i]);
          tmem_ld_32x32(tdP + lane_base + half * 32, raw);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) dv[half * 32 + i] = __uint_as_float(raw[i]);
        }
      }
      const int kbase = j * 64;
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        const bool valid = q_ok && (kbase + i <= qpos);
        const float pr = valid ? exp2f(sv[i] * p.scale2 - lse_r) : 0.0f;
        dv[i] = pr * (dv[i] - delta_r);
      }
      store_row64<T>(sdS, r, dv);
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(bar_p);
    }
    if (ok) ok = mbar_wait(bar_m2, (nkb - 1) & 1, wctx, kErrWaitAttn);
    if (ok) {
      tc_fence_after();
      T* drow = static_cast<T*>(p.dqkv) + (static_cast<long long>(qi) * p.b + bi) * p.ld_dqkv + hi * 3 * D;
#pragma unroll 1
      for (int ch = 0; ch < D / 32; ++ch) {
        uint32_t raw[32];
        __syncwarp();
        tmem_ld_32x32(tdQ + lane_base + ch * 32, raw);
        tmem_ld_wait();
        if (q_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 u;
            u.x = Elem<T>::pack2(__uint_as_float(raw[g * 8 + 0]) * p.scale, __uint_as_float(raw[g * 8 + 1]) * p.scale);
            u.y = Elem<T>::pack2(__uint_as_float(raw[g * 8 + 2]) * p.scale, __uint_as_float(raw[g * 8 + 3]) * p.scale);
            u.z = Elem<T>::pack2(__uint_as_float(raw[g * 8 + 4]) * p.scale, __uint_as_float(raw[g * 8 + 5]) * p.scale);
            u.w = Elem<T>::pack2(__uint_as_float(raw[g * 8 + 6]) * p.scale, __uint_as_float(raw[g * 8 + 7]) * p.scale);
            *reinterpret_cast<uint4*>(drow + ch * 32 + g * 8) = u;
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
  if (warp == 4) tmem_dealloc(tmem, kTmemCols);
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

template <int D> constexpr int fwd_smem() { return (D / 64) * (128 * 128 + 2 * 64 * 128) + 128 * 128 + 1024 + 256; }
template <int D> constexpr int dkdv_smem() { return (D / 64) * (2 * 128 * 128 + 4 * 64 * 128) + 2 * 128 * 128 + 1024 + 1024 + 256; }
template <int D> constexpr int dq_smem() { return (D / 64) * (2 * 128 * 128 + 4 * 64 * 128) + 128 * 128 + 1024 + 256; }

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
  kern<<<grid, kAttnThreads, fwd_smem<D>(), s>>>(tmQ, tmKV, p);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

template <typename T, int D>
static int attn_bwd_launch(const void* qkv, const void* o, const void* d_o, long long ld_do,
                           float* delta, const AttnParams& p, bool bf16, cudaStream_t s) {
  CUtensorMap tm128, tm64, tmdO64, tmdO128;
  if (!qkv_tmap(&tm128, qkv, D, p.b, p.h, p.c + p.t, 128, bf16) ||
      !qkv_tmap(&tm64, qkv, D, p.b, p.h, p.c + p.t, 64, bf16) ||
      !do_tmap(&tmdO64, d_o, ld_do, D, p.b, p.h, p.t, 64, bf16) ||
      !do_tmap(&tmdO128, d_o, ld_do, D, p.b, p.h, p.t, 128, bf16))
    return kErrDriver;
  {
    const long long warps = static_cast<long long>(p.t) * p.b * p.h;
    const int threads = 256;
    const int blocks = static_cast<int>((warps * 32 + threads - 1) / threads);
    attn_delta_kernel<T><<<blocks, threads, 0, s>>>(static_cast<const T*>(o), p.ld_o,
                                                    static_cast<const T*>(d_o), ld_do, delta, p.t,
                                                    p.b, p.h, D);
  }
  auto k1 = attn_bwd_dkdv_kernel<T, D>;
  auto k2 = attn_bwd_dq_kernel<T, D>;
  static bool cfg = false;
  if (!cfg) {
    if (!set_smem(k1, dkdv_smem<D>()) || !set_smem(k2, dq_smem<D>())) return kErrLaunch;
    cfg = true;
  }
  dim3 g1((p.c + p.t + 127) / 128, p.b * p.h);
  k1<<<g1, kAttnThreads, dkdv_smem<D>(), s>>>(tm128, tm64, tmdO64, p);
  dim3 g2((p.t + 127) / 128, p.b * p.h);
  k2<<<g2, kAttnThreads, dq_smem<D>(), s>>>(tm128, tm64, tmdO128, p);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

}  // namespace tp

using namespace tp;

static AttnParams base_params(int D, int b, int h, int t, int c, int* err) {
  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.t = t; p.c = c; p.b = b; p.h = h;
  p.scale = 1.0f / sqrtf(static_cast<float>(D));
  p.scale2 = p.scale * 1.4426950408889634f;
  p.err = err;
  return p;
}

// qkv: base of the full-length [L][b][h][3][D] buffer; rows [0, c+t) must be valid.
extern "C" int tp_attn_fwd(int dtype, int D, const void* qkv, int b, int h, int t, int c, void* o,
                           long long ld_o, float* lse2, long long lse_stride, int* err,
                           void* stream) {
  if ((D != 64 && D != 128) || t <= 0 || c < 0 || b <= 0 || h <= 0) return kErrBadArgument;
  if (ld_o % 8) return kErrBadArgument;
  AttnParams p = base_params(D, b, h, t, c, err);
  p.o = o; p.ld_o = ld_o; p.lse2 = lse2; p.lse_stride = lse_stride;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool bf16 = dtype == 1;
  if (D == 128) return bf16 ? attn_fwd_launch<__nv_bfloat16, 128>(qkv, p, true, s)
                            : attn_fwd_launch<__half, 128>(qkv, p, false, s);
  return bf16 ? attn_fwd_launch<__nv_bfloat16, 64>(qkv, p, true, s)
              : attn_fwd_launch<__half, 64>(qkv, p, false, s);
}

// o / d_o: this slice's [t*b][ld] attention output and its gradient; delta: fp32 [b*h*t]
// workspace; dkv_acc: persistent fp32 [b*h][dkv_rows][2][D] (dkv_rows >= c+t); dqkv: this slice's [t*b][ld_dqkv] output.
extern "C" int tp_attn_bwd(int dtype, int D, const void* qkv, int b, int h, int t, int c,
                           const void* o, long long ld_o, const void* d_o, long long ld_do,
                           const float* lse2, long long lse_stride, float* delta, float* dkv_acc,
                           long long dkv_rows, void* dqkv, long long ld_dqkv, int first, int* err, void* stream) {
  if ((D != 64 && D != 128) || t <= 0 || c < 0 || b <= 0 || h <= 0) return kErrBadArgument;
  if (ld_o % 8 || ld_do % 8 || ld_dqkv % 8) return kErrBadArgument;
  AttnParams p = base_params(D, b, h, t, c, err);
  p.o = const_cast<void*>(o); p.ld_o = ld_o;
  p.lse2 = const_cast<float*>(lse2); p.lse_stride = lse_stride;
  p.delta = delta; p.dkv_acc = dkv_acc; p.dkv_rows = dkv_rows; p.dqkv = dqkv; p.ld_dqkv = ld_dqkv; p.first = first;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool bf16 = dtype == 1;
  if (D == 128) return bf16 ? attn_bwd_launch<__nv_bfloat16, 128>(qkv, o, d_o, ld_do, delta, p, true, s)
                            : attn_bwd_launch<__half, 128>(qkv, o, d_o, ld_do, delta, p, false, s);
  return bf16 ? attn_bwd_launch<__nv_bfloat16, 64>(qkv, o, d_o, ld_do, delta, p, true, s)
              : attn_bwd_launch<__half, 64>(qkv, o, d_o, ld_do, delta, p, false, s);
}
