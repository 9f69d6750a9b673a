// Persistent warp-specialised GEMM for sm_100a: TMA -> shared-memory ring -> tcgen05.mma
// with fp32 accumulators in TMEM (double buffered) -> fused epilogue.
//
//   out[m][n] = epilogue( alpha * sum_k A(m,k) * B(n,k) )
//
// Operand storage (16-bit elements, fp16 or bf16):
//   a_mn = 0: A is [M][K] row-major (K contiguous);  a_mn = 1: A is stored [K][M] (M contiguous)
//   b_mn = 0: B is [N][K] row-major (a Linear weight); b_mn = 1: B is stored [K][N]
// which covers forward (0,0), data-gradient (0,1) and weight-gradient (1,1) products of a
// Linear layer without any transposed copies.
//
// Epilogue (all optional): + bias[n]; activation (ReLU / exact GeLU, optionally storing the
// pre-activation); + residual[m][n]; multiplication by the activation derivative evaluated
// on an auxiliary tensor (backward of the FFN nonlinearity); 16-bit or fp32 output; fp32
// output may accumulate (out += ...), which is how weight gradients of successive token
// slices add up in the main-gradient buffer.
//
// One CTA per SM, 192 threads: warp 0 = TMA producer, warp 1 = MMA issuer (owns TMEM),
// warps 2..5 = epilogue (one TMEM lane quarter each).
//
// Fused tensor-parallel all-reduce (template flag AR).  Every rank of a tensor-parallel group
// runs the same GEMM on its K shard; the partial products must be summed over ranks.  Instead
// of a separate collective, the kernel finishes the sum itself over NVLink peer memory:
//   A. each output tile has an owner rank (tile index modulo group size); the epilogue stores
//      the 16-bit partial tile into the owner's staging buffer and raises a per-(tile, source)
//      flag there (system-scope release);
//   B. after its own tiles, every CTA reduces the tiles its rank owns: waits for the flags of
//      all sources, sums the partials in fp32, adds bias and residual, and stores the result
//      into the output buffer of EVERY rank (peer stores), then raises a per-tile arrival flag
//      on every rank;
//   C. before exiting, the CTAs of a rank wait until all tiles have arrived locally.
// The transfer of a tile overlaps the math of later tiles.  All waits are bounded; flags carry a
// call counter ("epoch") so they never need clearing.  Peer buffers are plain device
// allocations mapped through CUDA IPC; only ordinary loads and stores touch peer memory.
#include "common.cuh"
#include "ptx.cuh"
#include "tile_order.h"

namespace tp {

struct GemmParams {
  int M, N, K;
  int num_m_tiles, num_tiles;
  // CTA-pair kernel: tile order (fields and meaning as in TileOrder, tile_order.h).  The
  // all-gather variant puts the row blocks whose operands are local first; the reduce-scatter
  // variant puts the row blocks this rank owns last, a whole phase after the peers produced
  // their share.
  int num_n_tiles, m_major, m_first, order_split, order_group, order_first_only, order_pipelined;
  // All-gather wait (CTA-pair kernel, A stored [M][K]): rows [s * ag_rows, (s + 1) * ag_rows) of A
  // were written into this GPU's memory by rank s; before loading rows of another rank the
  // producer waits until ag_flags[s] >= ag_epoch + *ag_epoch_base.  ag_flags == nullptr: no wait.
  const int* ag_flags;
  const int* ag_epoch_base;
  int ag_epoch, ag_rows, ag_rank;
  void* out;
  long long ldo;
  const void* bias;
  const void* residual;
  long long ldr;
  void* aux_out;
  const void* aux_in;
  long long ld_aux;
  float alpha;
  int act;         // 0 none, 1 relu, 2 gelu
  int dact;        // 0 none, 1 relu' (aux_in = activation output), 2 gelu' (aux_in = pre-activation)
  int accumulate;  // fp32 output only
  int* err;
  long long* trace;  // optional per-CTA phase stamps (trace builds of the kernel only)
  int prefetch;      // CTA-pair kernel: operand tiles are prefetched into L2 this many k-steps
                     // ahead of the loads that fill the ring (0 = off)
};

constexpr int kMaxTp = 8;

struct ArParams {
  int tp, rank;
  int epoch;                     // call index within the step; the kernel adds *epoch_base
  const int* epoch_base;         // device counter advanced once per step (graph-replay safe)
  int max_tiles;                 // capacity of the staging / flag arrays, in tiles
  int exchange;                  // CTA-pair kernel: every rank receives every partial tile and
                                 // reduces it itself (one NVLink hop instead of two)
  int rows_per_rank;             // reduce-scatter kernel: rank s owns rows [s * rows_per_rank, ...)
  void* stage[kMaxTp];           // per rank: [2 halves][tp sources][max_tiles][128][BN] 16-bit partials
                                 // (the second half is used by exchange mode only)
  int* flag_a[kMaxTp];           // per rank: [max_tiles][kMaxTp] partial-arrived flags
  int* flag_b[kMaxTp];           // per rank: [max_tiles] result-arrived flags
  void* out[kMaxTp];             // per rank: the output matrix (same offset in every pool)
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Spin until *p >= target; false on abort or after the wait limit.
__device__ __forceinline__ bool wait_flag(const int* p, int target, const WaitCtx& w, int code) {
  unsigned long long t0 = 0;
  unsigned spins = 0;
  while (ld_acquire_sys(p) < target) {
    if ((++spins & 0x3F) == 0) {
      if (*w.abort_smem) return false;
      // an earlier wait of this step already ran out (here or in an earlier kernel): the peers
      // are out of step for good, so do not spend another wait limit on every later flag
      if (w.err_global && *reinterpret_cast<volatile int*>(w.err_global) != 0) {
        *w.abort_smem = code;  // the CTA's own barrier waits end at once as well
        return false;
      }
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > g_wait_limit_ns) {
        report_timeout(w, code);
        return false;
      }
    }
  }
  return true;
}

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kGemmThreads = 192;
// staged output path of the epilogue (see EpiStage): two 32-row x 128-byte buffers per warp
constexpr int kEpiBufBytes = 4096;                      // 32 rows x 128 B
constexpr int kEpiBytesPerWarp = 2 * kEpiBufBytes;
constexpr int kEpiBytes = 4 * kEpiBytesPerWarp;         // four epilogue warps

// MT = number of 128-row sub-tiles of the CTA tile (1 or 2).  MT = 2 with BN = 256 gives a
// 256x256 tile: two MMAs per k-step share one B tile, which halves the shared-memory bytes
// fetched per FLOP (64 B/clk/SM at full rate instead of 96-128); both accumulators then fill
// the 512 TMEM columns, so the epilogue of a tile does not overlap the next tile's main loop.
template <int BN, int MT = 1, bool AR = false> struct GemmCfg {
  // the fused all-reduce variant gives one stage up for a [128][BN] 16-bit staging tile
  static constexpr int kStages = (MT == 2 ? 3 : (BN == 256 ? 4 : (BN == 128 ? 6 : 8))) - (AR ? 1 : 0);
  static constexpr int kArStageBytes = AR ? kBM * BN * 2 : 0;
  static constexpr int kABytes = MT * kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = BN == 64 ? 128 : 2 * BN;  // two accumulators, power of two
  static constexpr int kAccBuffers = MT == 2 ? 1 : 2;
  static constexpr int kEpiStageBytes = AR ? 0 : kEpiBytes;  // staged output path (not used with AR)
  static constexpr int kSmemBytes =
      kStages * kStageBytes + kArStageBytes + kEpiStageBytes + 1024 /*align*/ + 256 /*barriers*/;
};

// Not inlined on purpose: the epilogue applies them to 32 values per chunk, and 32 inlined erff
// expansions (twice, with the derivative) make the chunk code so large that the instruction
// fetch of the rarely executed epilogue dominates its run time.
__device__ __noinline__ float gelu_f(float z) {
  return 0.5f * z * (1.0f + erff(z * 0.70710678118654752f));
}
__device__ __noinline__ float gelu_grad_f(float z) {
  const float cdf = 0.5f * (1.0f + erff(z * 0.70710678118654752f));
  const float pdf = 0.3989422804014327f * __expf(-0.5f * z * z);
  return cdf + z * pdf;
}

// Staged output path of one epilogue warp.  A TMEM load hands every thread one ROW of the tile,
// so direct global stores would touch 32 different lines per instruction.  Instead the warp
// writes its 32 x 32 chunk into a private, swizzled shared-memory buffer (conflict free) and one
// lane stores the chunk with a single TMA tile store - or a TMA add-reduction when an fp32 output
// accumulates, which also removes the read of the old value.  The warp's buffers rotate, and
// the TMEM load of the next chunk is in flight while a chunk is processed.

// SM clock read that memory operations cannot be moved across (trace builds only)
__device__ __forceinline__ long long clock_ordered() {
  long long t;
  asm volatile("mov.u64 %0, %%clock64;" : "=l"(t)::"memory");
  return t;
}

struct EpiStage {
  uint8_t* buf;  // this warp's two buffers (1024-byte aligned)
  int issued;    // chunks stored so far by this warp
};

__device__ __forceinline__ void epi_drain(int lane) {
  if (lane == 0) bulk_wait<0>();
  __syncwarp();
}

// Fused epilogue of one 32-column chunk: r holds the fp32 accumulators of columns [n, n + 32)
// of row `row` (thread = row).  row0 is the first row of the warp's 32-row group (row0 < M);
// the caller has checked n < N.  t_next: TMEM address of the next chunk to load into r, or 0.  Rows >= M and columns >= N are clipped by the tile store.
template <typename T, bool OUT_F32, bool TRACE = false>
__device__ __forceinline__ void epilogue_chunk(const GemmParams& p, const CUtensorMap* tmO,
                                               EpiStage& es, uint32_t (&r)[32], long long row,
                                               bool row_ok, int n, int row0, int lane,
                                               uint32_t t_next, long long* cyc = nullptr,
                                               const T* part = nullptr, long long part_stride = 0,
                                               int n_src = 0, int self = 0) {
  const long long t_0 = TRACE ? clock_ordered() : 0;
  // Issue every global load of this 32-column chunk before any dependent math or store,
  // so the chunk pays one memory latency instead of one per 8-column group.
  bool gok[4];
  uint4 bv[4], rv[4], av[4];
#pragma unroll
  for (int g = 0; g < 4; ++g) gok[g] = n + g * 8 + 8 <= p.N;
  const uint4 zero4 = make_uint4(0, 0, 0, 0);
  if (p.bias) {
#pragma unroll
    for (int g = 0; g < 4; ++g)
      bv[g] = gok[g] ? __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(p.bias) + n + g * 8)) : zero4;
  }
  if (p.residual) {
#pragma unroll
    for (int g = 0; g < 4; ++g)
      rv[g] = (gok[g] && row_ok)
                  ? __ldcg(reinterpret_cast<const uint4*>(static_cast<const T*>(p.residual) + row * p.ldr + n + g * 8))
                  : zero4;
  }
  if (p.dact) {
#pragma unroll
    for (int g = 0; g < 4; ++g)
      av[g] = (gok[g] && row_ok)
                  ? __ldcg(reinterpret_cast<const uint4*>(static_cast<const T*>(p.aux_in) + row * p.ld_aux + n + g * 8))
                  : zero4;
  }
  // Reduce-scatter: the other ranks' 16-bit partials of this chunk (thread = row, 64 contiguous
  // bytes per source in this rank's staging buffer); the first source is fetched here with the
  // other operands, further ones (groups of more than two ranks) in a loop below.
  uint4 pa[4];
  int src_a = -1;
  if (part) {
    src_a = self == 0 ? 1 : 0;
#pragma unroll
    for (int g = 0; g < 4; ++g)
      pa[g] = __ldcg(reinterpret_cast<const uint4*>(part + src_a * part_stride + g * 8));
  }
  // A tile store reads its source a good thousand cycles after it was issued, so the buffers
  // rotate: four 2 KB buffers for 16-bit output, two 4 KB buffers for fp32.  The buffer about
  // to be overwritten was the source of the store issued kBufs chunks ago.
  constexpr int kBufs = OUT_F32 ? 2 : 4;
  uint8_t* sb = es.buf + (es.issued % kBufs) * (kEpiBytesPerWarp / kBufs);
  if (es.issued >= kBufs) {
    if (lane == 0) bulk_wait_read<kBufs - 1>();
    __syncwarp();
  }
  const long long t_1 = TRACE ? clock_ordered() : 0;
  // trace builds: a zero the compiler cannot see through ties the math below to the clock read
  const uint32_t tz = TRACE ? static_cast<uint32_t>(static_cast<unsigned long long>(t_1) >> 63) : 0u;
  // One pass per fused operation over all 32 values: one uniform branch per pass and 32
  // independent instructions inside it (a lone warp per scheduler needs the ILP).
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j] + tz);
  // r is free again: start the TMEM load of the next chunk (t_next = 0: there is none).  The
  // empty asm keeps the copies above ahead of the load that overwrites their source.
  asm volatile("" ::: "memory");
  if (t_next) tmem_ld_32x32(t_next, r);
  if (p.alpha != 1.0f) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] *= p.alpha;
  }
  if (part) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const uint32_t aw[4] = {pa[g].x, pa[g].y, pa[g].z, pa[g].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 fa = Elem<T>::unpack2(aw[j]);
        v[g * 8 + 2 * j] += fa.x;
        v[g * 8 + 2 * j + 1] += fa.y;
      }
    }
#pragma unroll 1
    for (int q = src_a + 1; q < n_src; ++q) {  // groups of more than two ranks
      if (q == self) continue;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const uint4 u = __ldcg(reinterpret_cast<const uint4*>(part + q * part_stride + g * 8));
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = Elem<T>::unpack2(w[j]);
          v[g * 8 + 2 * j] += f.x;
          v[g * 8 + 2 * j + 1] += f.y;
        }
      }
    }
  }
  if (p.bias) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const uint32_t bw[4] = {bv[g].x, bv[g].y, bv[g].z, bv[g].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = Elem<T>::unpack2(bw[j]);
        v[g * 8 + 2 * j] += f.x;
        v[g * 8 + 2 * j + 1] += f.y;
      }
    }
  }
  if (p.act == 2) {
    if (p.aux_out && row_ok) {
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        if (!gok[g]) continue;
        uint4 zv;
        zv.x = Elem<T>::pack2(v[g * 8 + 0], v[g * 8 + 1]);
        zv.y = Elem<T>::pack2(v[g * 8 + 2], v[g * 8 + 3]);
        zv.z = Elem<T>::pack2(v[g * 8 + 4], v[g * 8 + 5]);
        zv.w = Elem<T>::pack2(v[g * 8 + 6], v[g * 8 + 7]);
        __stcg(reinterpret_cast<uint4*>(static_cast<T*>(p.aux_out) + row * p.ld_aux + n + g * 8), zv);
      }
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = gelu_f(v[j]);
  } else if (p.act == 1) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.0f);
  }
  if (p.residual) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const uint32_t rw[4] = {rv[g].x, rv[g].y, rv[g].z, rv[g].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = Elem<T>::unpack2(rw[j]);
        v[g * 8 + 2 * j] += f.x;
        v[g * 8 + 2 * j + 1] += f.y;
      }
    }
  }
  if (p.dact) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const uint32_t aw[4] = {av[g].x, av[g].y, av[g].z, av[g].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = Elem<T>::unpack2(aw[j]);
        if (p.dact == 1) {
          v[g * 8 + 2 * j] = f.x > 0.0f ? v[g * 8 + 2 * j] : 0.0f;
          v[g * 8 + 2 * j + 1] = f.y > 0.0f ? v[g * 8 + 2 * j + 1] : 0.0f;
        } else {
          v[g * 8 + 2 * j] *= gelu_grad_f(f.x);
          v[g * 8 + 2 * j + 1] *= gelu_grad_f(f.y);
        }
      }
    }
  }
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    if (OUT_F32) {
      // 128-byte rows, 128-byte swizzle: 16-byte chunk index ^= row & 7
      uint8_t* rowp = sb + lane * 128;
      *reinterpret_cast<float4*>(rowp + (((2 * g) ^ (lane & 7)) << 4)) =
          make_float4(v[g * 8 + 0], v[g * 8 + 1], v[g * 8 + 2], v[g * 8 + 3]);
      *reinterpret_cast<float4*>(rowp + (((2 * g + 1) ^ (lane & 7)) << 4)) =
          make_float4(v[g * 8 + 4], v[g * 8 + 5], v[g * 8 + 6], v[g * 8 + 7]);
    } else {
      // 64-byte rows, 64-byte swizzle: 16-byte chunk index ^= (row >> 1) & 3
      uint4 ov;
      ov.x = Elem<T>::pack2(v[g * 8 + 0], v[g * 8 + 1]);
      ov.y = Elem<T>::pack2(v[g * 8 + 2], v[g * 8 + 3]);
      ov.z = Elem<T>::pack2(v[g * 8 + 4], v[g * 8 + 5]);
      ov.w = Elem<T>::pack2(v[g * 8 + 6], v[g * 8 + 7]);
      *reinterpret_cast<uint4*>(sb + lane * 64 + ((g ^ ((lane >> 1) & 3)) << 4)) = ov;
    }
  }
  const long long t_2 = TRACE ? clock_ordered() : 0;
  fence_proxy_async();
  __syncwarp();
  if (lane == 0) {
    if (OUT_F32 && p.accumulate) tma_reduce_add_2d(tmO, sb, n, row0);
    else tma_store_2d(tmO, sb, n, row0);
    bulk_commit();
  }
  ++es.issued;
  if (TRACE) {
    cyc[0] += t_1 - t_0;        // loads issued, staging buffer free
    cyc[1] += t_2 - t_1;        // math and shared-memory writes
    cyc[2] += clock_ordered() - t_2;  // proxy fence, tile store issued
  }
}

// (Output-tile coordinates of the CTA-pair kernel: pair_tile_coords in tile_order.h.)

// Epilogue of one warp's 32 rows over `nc` 32-column chunks of an accumulator at TMEM address
// `t_acc` (lane quarter already applied); the warp takes chunks c_first, c_first + c_step, ...
// The chunk code exists once (it is large); the TMEM
// load of chunk c + 1 is issued from inside it as soon as chunk c's values have been copied out
// of the load registers.
template <typename T, bool OUT_F32, bool TRACE = false>
__device__ __forceinline__ void epilogue_rows(const GemmParams& p, const CUtensorMap* tmO,
                                              EpiStage& es, uint32_t t_acc, int nc, int row0, int n0,
                                              int lane, int c_first = 0, int c_step = 1,
                                              long long* cyc = nullptr, const T* part = nullptr,
                                              long long part_stride = 0, int n_src = 0, int self = 0) {
  const long long row = row0 + lane;
  const bool row_ok = row < p.M;
  uint32_t r[32];
  __syncwarp();
  if (c_first >= nc) return;
  tmem_ld_32x32(t_acc + c_first * 32, r);
#pragma unroll 1
  for (int c = c_first; c < nc; c += c_step) {
    tmem_ld_wait();
    epilogue_chunk<T, OUT_F32, TRACE>(p, tmO, es, r, row, row_ok, n0 + c * 32, row0, lane,
                                      c + c_step < nc ? t_acc + (c + c_step) * 32 : 0u, cyc,
                                      part ? part + c * 4096 : nullptr, part_stride, n_src, self);
  }
}

template <typename T, int BN, bool A_MN, bool B_MN, bool OUT_F32, bool AR = false, int MT = 1>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmO, const GemmParams p, const ArParams ar) {
  using Cfg = GemmCfg<BN, MT, AR>;
  constexpr int S = Cfg::kStages;
  constexpr int BM = MT * kBM;
  constexpr int NACC = Cfg::kAccBuffers;
  static_assert(!(AR && MT != 1), "the fused all-reduce path uses 128-row tiles");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* ar_tile = smem + S * Cfg::kStageBytes;  // AR only: row-major [128][BN] partial tile
  uint8_t* epi_smem = smem + S * Cfg::kStageBytes + Cfg::kArStageBytes;  // non-AR: output staging
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + Cfg::kEpiStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + S;
  uint64_t* tfull = bars + 2 * S;
  uint64_t* tempty = bars + 2 * S + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitCtx wctx{abort_flag, p.err};

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    if (!AR) prefetch_tmap(&tmO);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();  // set-up done; from here on the predecessor's results are read

  const int num_kb = (p.K + kBK - 1) / kBK;
  const int ar_epoch = AR ? (ar.epoch + (ar.epoch_base ? *ar.epoch_base : 0)) : 0;

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
        const int m0 = (tile % p.num_m_tiles) * BM;
        const int n0 = (tile / p.num_m_tiles) * BN;
        bool ok = true;
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          ok = mbar_wait(&empty[stage], phase ^ 1, wctx, kErrWaitProducer);
          if (!ok) break;
          uint8_t* sA = smem + stage * Cfg::kStageBytes;
          uint8_t* sB = sA + Cfg::kABytes;
          mbar_expect_tx(&full[stage], Cfg::kStageBytes);
          if (!A_MN) {
            tma_load_2d(sA, &tmA, &full[stage], kb * kBK, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d(sA + c * (kBK * 128), &tmA, &full[stage], m0 + c * 64, kb * kBK);
          }
          if (!B_MN) {
            tma_load_2d(sB, &tmB, &full[stage], kb * kBK, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sB + c * (kBK * 128), &tmB, &full[stage], n0 + c * 64, kb * kBK);
          }
          if (++stage == S) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_f16(Elem<T>::fmt, A_MN ? 1 : 0, B_MN ? 1 : 0, kBM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++it) {
        const int acc = it % NACC;
        const uint32_t acc_phase = (it / NACC) & 1;
        ok = mbar_wait(&tempty[acc], acc_phase ^ 1, wctx, kErrWaitTmemEmpty);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(&full[stage], phase, wctx, kErrWaitMma);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_base = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t b_base = a_base + Cfg::kABytes;
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t db = B_MN ? umma_desc_sw128(b_base + k * 2048, kBK * 128, 1024)
                                     : umma_desc_sw128(b_base + k * 32, 16, 1024);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              // sub-tile mt: rows [128 mt, 128 mt + 128) of the A tile (K-major: 128 rows of
              // 128 B; M-major: two 64-wide chunks of kBK rows each)
              const uint32_t a_sub = a_base + mt * (A_MN ? 2 * kBK * 128 : kBM * 128);
              const uint64_t da = A_MN ? umma_desc_sw128(a_sub + k * 2048, kBK * 128, 1024)
                                       : umma_desc_sw128(a_sub + k * 32, 16, 1024);
              umma_f16(d_tmem + mt * BN, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
            }
          }
          umma_commit(&empty[stage]);
          if (++stage == S) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
      }
    }
  } else {
    const int quarter = warp & 3;  // TMEM lane quarter this warp may access
    const int row_in_tile = quarter * 32 + lane;
    EpiStage es{epi_smem + quarter * kEpiBytesPerWarp, 0};
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++it) {
      const int acc = it % NACC;
      const uint32_t acc_phase = (it / NACC) & 1;
      const int m0 = (tile % p.num_m_tiles) * BM;
      const int n0 = (tile / p.num_m_tiles) * BN;
      ok = mbar_wait(&tfull[acc], acc_phase, wctx, kErrWaitEpilogue);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      if (AR) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t r[32];
          __syncwarp();
          tmem_ld_32x32(t_acc + c0, r);
          tmem_ld_wait();
          // phase A, step 1: 16-bit partial of this chunk into the CTA's staging tile (row-major)
          T* dst = reinterpret_cast<T*>(ar_tile) + row_in_tile * BN + c0;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 ov;
            ov.x = Elem<T>::pack2(__uint_as_float(r[g * 8 + 0]) * p.alpha, __uint_as_float(r[g * 8 + 1]) * p.alpha);
            ov.y = Elem<T>::pack2(__uint_as_float(r[g * 8 + 2]) * p.alpha, __uint_as_float(r[g * 8 + 3]) * p.alpha);
            ov.z = Elem<T>::pack2(__uint_as_float(r[g * 8 + 4]) * p.alpha, __uint_as_float(r[g * 8 + 5]) * p.alpha);
            ov.w = Elem<T>::pack2(__uint_as_float(r[g * 8 + 6]) * p.alpha, __uint_as_float(r[g * 8 + 7]) * p.alpha);
            *reinterpret_cast<uint4*>(dst + g * 8) = ov;
          }
        }
      } else {
        // columns of this tile inside the matrix, in 32-column chunks (warp-uniform)
        const int nc = (min(BN, p.N - n0) + 31) / 32;
#pragma unroll 1
        for (int mt = 0; mt < MT; ++mt) {
          const int row0 = m0 + mt * kBM + quarter * 32;
          if (row0 >= p.M) continue;  // warp-uniform: nothing to store
          epilogue_rows<T, OUT_F32>(p, &tmO, es, t_acc + mt * BN, nc, row0, n0, lane);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      if (AR) {
        // phase A, step 2: the staging tile is one contiguous block in the owner's memory, so
        // the 128 epilogue threads copy it with fully coalesced 16-byte stores (512 contiguous
        // bytes per warp instruction over NVLink), then one thread publishes the tile.  The
        // release store is cumulative over the writes ordered before it by the barrier.
        asm volatile("bar.sync 1, 128;" ::: "memory");
        // checked build: the tile's slot in the owner's staging and flag arrays exists
        const bool slot_ok = TP_CHECK(tile >= 0 && tile < ar.max_tiles && ar.tp <= kMaxTp, p.err,
                                      kErrCheckStaging);
        if (slot_ok) {
          const int owner = tile % ar.tp;
          uint4* dst = reinterpret_cast<uint4*>(
              static_cast<T*>(ar.stage[owner]) +
              (static_cast<long long>(ar.rank) * ar.max_tiles + tile) * kBM * BN);
          const uint4* src = reinterpret_cast<const uint4*>(ar_tile);
          const int e = threadIdx.x - 64;
#pragma unroll
          for (int k = 0; k < kBM * BN * 2 / 16 / 128; ++k) dst[e + k * 128] = src[e + k * 128];
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64 && slot_ok)
          st_release_sys(ar.flag_a[tile % ar.tp] + static_cast<long long>(tile) * kMaxTp + ar.rank, ar_epoch);
      }
    }
    if (!AR) epi_drain(lane);  // the staging buffers must outlive the stores that read them
  }

  if (AR) {
    __syncthreads();
    __shared__ int s_ok;
    // phase B: reduce the tiles this rank owns and push the result to every rank
    const int n_owned = (p.num_tiles - ar.rank + ar.tp - 1) / ar.tp;
    for (int j = blockIdx.x; j < n_owned; j += gridDim.x) {
      const int tile = j * ar.tp + ar.rank;
      if (!TP_CHECK(tile >= 0 && tile < ar.max_tiles, p.err, kErrCheckStaging)) continue;
      if (threadIdx.x == 0) {
        bool ok = true;
        for (int src = 0; src < ar.tp && ok; ++src)
          ok = wait_flag(ar.flag_a[ar.rank] + static_cast<long long>(tile) * kMaxTp + src, ar_epoch, wctx,
                         kErrWaitPeer);
        s_ok = ok ? 1 : 0;
      }
      __syncthreads();
      if (s_ok) {
        const int m0 = (tile % p.num_m_tiles) * kBM;
        const int n0 = (tile / p.num_m_tiles) * BN;
        const T* stage = static_cast<const T*>(ar.stage[ar.rank]);
        for (int v = threadIdx.x; v < kBM * BN / 8; v += kGemmThreads) {
          const int rr = v / (BN / 8), cc = (v % (BN / 8)) * 8;
          const long long row = m0 + rr;
          const int col = n0 + cc;
          if (row >= p.M || col + 8 > p.N) continue;
          float acc8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          for (int src = 0; src < ar.tp; ++src) {
            const uint4 u = __ldcg(reinterpret_cast<const uint4*>(
                stage + ((static_cast<long long>(src) * ar.max_tiles + tile) * kBM + rr) * BN + cc));
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 f = Elem<T>::unpack2(w[q]);
              acc8[2 * q] += f.x;
              acc8[2 * q + 1] += f.y;
            }
          }
          if (p.bias) {
            const uint4 u = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(p.bias) + col));
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 f = Elem<T>::unpack2(w[q]);
              acc8[2 * q] += f.x;
              acc8[2 * q + 1] += f.y;
            }
          }
          if (p.residual) {
            const uint4 u = __ldcg(reinterpret_cast<const uint4*>(static_cast<const T*>(p.residual) + row * p.ldr + col));
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 f = Elem<T>::unpack2(w[q]);
              acc8[2 * q] += f.x;
              acc8[2 * q + 1] += f.y;
            }
          }
          uint4 ov;
          ov.x = Elem<T>::pack2(acc8[0], acc8[1]);
          ov.y = Elem<T>::pack2(acc8[2], acc8[3]);
          ov.z = Elem<T>::pack2(acc8[4], acc8[5]);
          ov.w = Elem<T>::pack2(acc8[6], acc8[7]);
          for (int dst = 0; dst < ar.tp; ++dst)
            *reinterpret_cast<uint4*>(static_cast<T*>(ar.out[dst]) + row * p.ldo + col) = ov;
        }
      }
      __syncthreads();
      if (s_ok && threadIdx.x < ar.tp) st_release_sys(ar.flag_b[threadIdx.x] + tile, ar_epoch);
    }
    // phase C: every tile of the output must have arrived in this rank's memory
    for (int tile = blockIdx.x * kGemmThreads + threadIdx.x; tile < p.num_tiles;
         tile += gridDim.x * kGemmThreads)
      if (TP_CHECK(tile < ar.max_tiles, p.err, kErrCheckStaging))
        wait_flag(ar.flag_b[ar.rank] + tile, ar_epoch, wctx, kErrWaitPeer);
  }

  // teardown: on an aborted run give in-flight bulk copies time to land before the CTA's
  // shared memory is released, then free TMEM.
  __syncthreads();
  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

template <typename T, int BN, bool A_MN, bool B_MN, bool OUT_F32, bool AR = false, int MT = 1>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmO,
                       const GemmParams& p, cudaStream_t stream, const ArParams* arp = nullptr) {
  using Cfg = GemmCfg<BN, MT, AR>;
  auto kern = gemm_kernel<T, BN, A_MN, B_MN, OUT_F32, AR, MT>;
  ArParams ar;
  if (arp) ar = *arp;
  else { ar.tp = 0; ar.exchange = 0; ar.rows_per_rank = 0; }
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) !=
        cudaSuccess)
      return kErrLaunch;
    configured = true;
  }
  int grid = p.num_tiles < num_sms() ? p.num_tiles : num_sms();
  return launch_pdl(kern, dim3(grid), dim3(kGemmThreads), Cfg::kSmemBytes, stream, 1, tmA, tmB, tmO, p, ar) ==
                 cudaSuccess
             ? kOk
             : kErrLaunch;
}

template <typename T, int BN, int MT = 1>
static int dispatch_layout(int a_mn, int b_mn, int out_f32, const CUtensorMap& tmA,
                           const CUtensorMap& tmB, const CUtensorMap& tmO, const GemmParams& p,
                           cudaStream_t s) {
  if (!a_mn && !b_mn && !out_f32) return launch_gemm<T, BN, false, false, false, false, MT>(tmA, tmB, tmO, p, s);
  if (!a_mn && b_mn && !out_f32) return launch_gemm<T, BN, false, true, false, false, MT>(tmA, tmB, tmO, p, s);
  if (a_mn && b_mn && out_f32) return launch_gemm<T, BN, true, true, true, false, MT>(tmA, tmB, tmO, p, s);
  if (MT == 1) {  // rarely used layouts: only the 128-row tile is instantiated
    if (!a_mn && !b_mn && out_f32) return launch_gemm<T, BN, false, false, true>(tmA, tmB, tmO, p, s);
    if (a_mn && b_mn && !out_f32) return launch_gemm<T, BN, true, true, false>(tmA, tmB, tmO, p, s);
  }
  return kErrBadArgument;
}

// ---------------------------------------------------------------------------------------------
// CTA-pair variant (tcgen05 cta_group::2).  A cluster of two CTAs, one per SM of a TPC, owns a
// 256 x BN output tile: CTA r of the pair loads rows [128 r, 128 r + 128) of the A tile and
// rows [BN/2 r, BN/2 r + BN/2) of the B tile into its own shared memory and keeps 128 lanes x
// BN columns of the fp32 accumulator in its own TMEM; the leader CTA (rank 0) issues one MMA
// per k16 step for both.  Per SM and k16 step the tensor core then reads 4 KB of A and only
// BN/2 rows of B (4 KB for BN = 256) while TMA writes the same amount: 64 + 64 B/clk, inside the
// 128 B/clk a shared memory delivers, where a lone CTA with a 128 x 256 tile needs 96 + 96.
// Unlike the 256 x 256 single-CTA tile the accumulator is still double buffered (2 x BN columns
// per CTA), so the epilogue of a tile overlaps the main loop of the next one.
//
// Synchronisation across the pair:
//   full[s]   lives in the leader; both CTAs' TMA loads count their bytes on it;
//   empty[s]  one per CTA, both signalled by one tcgen05.commit of the leader;
//   tfull[a]  one per CTA (epilogue warps of each CTA wait on their own), same commit form;
//   tempty[a] lives in the leader, 16 arrivals: the 8 epilogue warps of each CTA.
// Ten warps: 0 = TMA producer, 1 = MMA issuer, 2..9 = epilogue.  A lone warp per scheduler
// runs the long straight-line epilogue code at only one instruction per 4-5 cycles (it is bound
// by instruction fetch, not by TMEM or shared memory), so two warps share each TMEM lane quarter
// and take alternate 32-column chunks; that halves the exposed epilogue of a CTA's last tile.
constexpr int kPairThreads = 320;
constexpr int kPairEpiWarps = 8;

template <int BN> struct PairCfg {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = (BN / 2) * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = BN == 256 ? 5 : 6;
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kEpiStageBytes = kPairEpiWarps * kEpiBytesPerWarp;
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiStageBytes + 1024 /*align*/ + 256 /*barriers*/;
};

// TRACE = true additionally records, per CTA, SM-clock stamps of the pipeline phases into
// p.trace[blockIdx.x * kTraceSlots ...] (see the slot list at tp_gemm_trace).
constexpr int kTraceSlots = 24;

// Phase B of the fused all-reduce for one 128 x BN tile this rank owns (staging layout of the
// CTA-pair kernel: 16 blocks [column chunk][lane quarter] of [32 rows][32 columns]): sum the
// partials of all ranks, add bias and residual, store the result into every rank's output.
// Called by `nthreads` threads with tid in [0, nthreads) after the tile's flags were observed.
// local_only: exchange mode, the other ranks reduce the tile themselves.
template <typename T, int BN>
__device__ __forceinline__ void ar_reduce_tile(const GemmParams& p, const ArParams& ar, int tile,
                                               int num_m128, int tid, int nthreads, bool local_only,
                                               long long stage_half) {
  const int m0 = (tile % num_m128) * kBM;
  const int n0 = (tile / num_m128) * BN;
  const T* stage = static_cast<const T*>(ar.stage[ar.rank]) + stage_half;
  // Four 16-byte vectors per thread and round: all loads of a round are issued before any of
  // them is used, so a tile costs two or three memory round trips instead of one per vector.
  constexpr int kBatch = 4;
  constexpr int kVecs = kBM * BN / 8;
  const uint4 zero4 = make_uint4(0, 0, 0, 0);
  for (int base = 0; base < kVecs; base += nthreads * kBatch) {
    uint4 part[kBatch][kMaxTp > 4 ? 4 : kMaxTp];  // up to 4 sources per pass (see below)
    uint4 bias4[kBatch], res4[kBatch];
    float acc[kBatch][8];
    bool ok[kBatch];
    long long row[kBatch];
    int col[kBatch], off[kBatch];
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
      const int v = base + tid + k * nthreads;
      const int rr = v / (BN / 8), c8 = v % (BN / 8);  // row in tile, 8-column group
      row[k] = m0 + rr;
      col[k] = n0 + c8 * 8;
      ok[k] = v < kVecs && row[k] < p.M && col[k] + 8 <= p.N;
      off[k] = ((c8 >> 2) * 4 + (rr >> 5)) * 1024 + (rr & 31) * 32 + (c8 & 3) * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[k][j] = 0.0f;
    }
    for (int s0 = 0; s0 < ar.tp; s0 += 4) {  // sources in passes of four
#pragma unroll
      for (int k = 0; k < kBatch; ++k)
#pragma unroll
        for (int q = 0; q < 4; ++q)
          part[k][q] = (ok[k] && s0 + q < ar.tp)
                           ? __ldcg(reinterpret_cast<const uint4*>(
                                 stage + (static_cast<long long>(s0 + q) * ar.max_tiles + tile) * (kBM * BN) + off[k]))
                           : zero4;
      if (s0 == 0) {
#pragma unroll
        for (int k = 0; k < kBatch; ++k) {
          bias4[k] = (ok[k] && p.bias)
                         ? __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(p.bias) + col[k]))
                         : zero4;
          res4[k] = (ok[k] && p.residual)
                        ? __ldcg(reinterpret_cast<const uint4*>(static_cast<const T*>(p.residual) + row[k] * p.ldr + col[k]))
                        : zero4;
        }
      }
#pragma unroll
      for (int k = 0; k < kBatch; ++k)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t w[4] = {part[k][q].x, part[k][q].y, part[k][q].z, part[k][q].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = Elem<T>::unpack2(w[j]);
            acc[k][2 * j] += f.x;
            acc[k][2 * j + 1] += f.y;
          }
        }
    }
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
      if (!ok[k]) continue;
      const uint32_t bw[4] = {bias4[k].x, bias4[k].y, bias4[k].z, bias4[k].w};
      const uint32_t rw[4] = {res4[k].x, res4[k].y, res4[k].z, res4[k].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 fb = Elem<T>::unpack2(bw[j]);
        const float2 fr = Elem<T>::unpack2(rw[j]);
        acc[k][2 * j] += fb.x + fr.x;
        acc[k][2 * j + 1] += fb.y + fr.y;
      }
      uint4 ov;
      ov.x = Elem<T>::pack2(acc[k][0], acc[k][1]);
      ov.y = Elem<T>::pack2(acc[k][2], acc[k][3]);
      ov.z = Elem<T>::pack2(acc[k][4], acc[k][5]);
      ov.w = Elem<T>::pack2(acc[k][6], acc[k][7]);
      if (local_only) {
        __stcg(reinterpret_cast<uint4*>(static_cast<T*>(ar.out[ar.rank]) + row[k] * p.ldo + col[k]), ov);
      } else {
        for (int dst = 0; dst < ar.tp; ++dst)
          *reinterpret_cast<uint4*>(static_cast<T*>(ar.out[dst]) + row[k] * p.ldo + col[k]) = ov;
      }
    }
  }
}

// AR = true fuses the tensor-parallel all-reduce exactly as gemm_kernel does (phases A-C of the
// file comment), with 128 x 128 all-reduce tiles: each CTA of a pair owns the flags and staging
// of its own 128 rows, so no flag needs a barrier across the pair.  In the owner's staging
// buffer a tile is stored as 16 blocks [column chunk c][lane quarter q] of [32 rows][32 columns];
// an epilogue warp produces exactly one such 2 KB block per chunk and copies it with fully
// coalesced 16-byte peer stores.
//
// RS = true fuses a reduce-scatter over the rows instead: rank s ends with rows
// [s * rows_per_rank, (s + 1) * rows_per_rank) of the summed product (rows_per_rank a multiple of
// 32).  An epilogue warp whose 32 rows belong to another rank pushes its chunks to that rank's
// staging buffer exactly as in phase A above; an extra warp (warp 10) publishes a 128-row block
// once all eight epilogue warps have stored their part, so no epilogue warp ever waits for the
// NVLink round trip of a system-scope release.  A warp whose rows belong to this rank waits for
// the other ranks' partials of its block and adds them, in fp32, to its accumulator inside the
// regular epilogue (bias, residual, staged TMA store).  With m_major tile order and the row
// blocks of this rank visited last, the partials have arrived long before they are needed and
// nothing follows the last tile: no second hop, no result flags.
template <typename T, int BN, bool A_MN, bool B_MN, bool OUT_F32, bool TRACE = false, bool AR = false,
          bool RS = false>
__global__ void __launch_bounds__(kPairThreads + (RS ? 32 : 0), 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmO, const GemmParams p, const ArParams ar) {
  static_assert(!AR || (BN == 128 && !OUT_F32 && !TRACE), "fused all-reduce: 256 x 128 pair tiles, 16-bit output");
  static_assert(!RS || (BN == 128 && !OUT_F32 && !TRACE && !AR && !A_MN), "fused reduce-scatter: 256 x 128 pair tiles, 16-bit output");
  using Cfg = PairCfg<BN>;
  constexpr int S = Cfg::kStages;
  constexpr int HB = BN / 2;  // B rows held by one CTA
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* epi_smem = smem + S * Cfg::kStageBytes;  // output staging of the epilogue warps
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + Cfg::kEpiStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + S;
  uint64_t* tfull = bars + 2 * S;
  uint64_t* tempty = bars + 2 * S + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* s_ready = reinterpret_cast<volatile int*>(tmem_slot + 2);  // AR: owned tile ready?
  volatile int* s_next = reinterpret_cast<volatile int*>(tmem_slot + 3);   // AR: next owned tile
  uint64_t* pub_full = bars + 2 * S + 6;                                    // RS: block stored by all warps
  volatile int* pub_done = reinterpret_cast<volatile int*>(bars + 2 * S + 8);  // RS: blocks published

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();   // 0 = leader
  long long* tr = TRACE ? p.trace + static_cast<long long>(blockIdx.x) * kTraceSlots : nullptr;
  if (TRACE && threadIdx.x == 0) tr[0] = clock64();
  const int pair = blockIdx.x >> 1;
  const int npairs = gridDim.x >> 1;
  const WaitCtx wctx{abort_flag, p.err};

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 2 * kPairEpiWarps);
    }
    *abort_flag = 0;
    *s_ready = 0;
    *s_next = (AR && ar.exchange) ? 0 : static_cast<int>(blockIdx.x);
    if (RS) {
      mbar_init(&pub_full[0], kPairEpiWarps);
      mbar_init(&pub_full[1], kPairEpiWarps);
      *pub_done = 0;
    }
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    prefetch_tmap(&tmO);
  }
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before any remote arrival
  pdl_wait();          // set-up done; from here on the predecessor's results are read
  // The producer warp starts loading at once; the other five warps meet again after the TMEM
  // allocation (named barrier 1, 288 threads).
  uint32_t tmem_base = 0;
  if (warp >= 1 && warp < 10) {
    if (warp == 1) {
      tmem_alloc_pair(tmem_slot, Cfg::kTmemCols);
      tmem_relinquish_pair();
    }
    tc_fence_before();
    asm volatile("bar.sync 1, 288;" ::: "memory");
    tc_fence_after();
    tmem_base = *tmem_slot;
  }
  const int num_kb = (p.K + kBK - 1) / kBK;
  const int ar_epoch = (AR || RS) ? (ar.epoch + (ar.epoch_base ? *ar.epoch_base : 0)) : 0;
  const int num_m128 = (p.M + kBM - 1) / kBM;  // AR: 128-row tiles of the output
  // Exchange mode and the reduce-scatter have no hand-shake after the reduction, so a rank may
  // start its next call while a peer still reads this call's partials: calls alternate between
  // two staging halves.
  const long long stage_half =
      (((AR && ar.exchange) || RS) && (ar_epoch & 1)) ? static_cast<long long>(ar.tp) * ar.max_tiles * (kBM * BN) : 0;
  if (TRACE && threadIdx.x == 0) tr[1] = clock64();

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long stall = 0;
      unsigned ag_seen = 0;  // ranks whose rows are known to have arrived
      for (int tile = pair; tile < p.num_tiles && ok; tile += npairs) {
        int m_idx, n_idx;
        pair_tile_coords(p, tile, m_idx, n_idx);
        const int m0 = m_idx * (2 * kBM) + static_cast<int>(cta) * kBM;
        const int n0 = n_idx * BN + static_cast<int>(cta) * HB;
        if (!A_MN && p.ag_flags != nullptr && m0 < p.M) {
          const int last_row = min(m0 + kBM, p.M) - 1;
          const int target = p.ag_epoch + (p.ag_epoch_base ? *p.ag_epoch_base : 0);
          bool waited = false;
          for (int src = m0 / p.ag_rows; src <= last_row / p.ag_rows && ok; ++src) {
            if (src == p.ag_rank || (ag_seen >> src) & 1u) continue;
            if (!TP_CHECK(src >= 0 && src < kMaxTp, p.err, kErrCheckPeer)) continue;
            ok = wait_flag(p.ag_flags + src, target, wctx, kErrWaitPeer);
            ag_seen |= 1u << src;
            waited = true;
          }
          if (!ok) break;
          // the rows were written by generic-proxy stores of another GPU; the loads below go
          // through the async proxy
          if (waited) asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          const long long t_w = TRACE ? clock64() : 0;
          ok = mbar_wait(&empty[stage], phase ^ 1, wctx, kErrWaitProducer);
          if (!ok) break;
          if (TRACE) stall += clock64() - t_w;
          uint8_t* sA = smem + stage * Cfg::kStageBytes;
          uint8_t* sB = sA + Cfg::kABytes;
          if (cta == 0) mbar_expect_tx(&full[stage], 2 * Cfg::kStageBytes);
          if (p.prefetch > 0 && kb + p.prefetch < num_kb) {
            // operands that come from DRAM (weights of a step are cold in L2) have a latency
            // the ring alone cannot cover; an L2 prefetch further ahead does
            const int kp = (kb + p.prefetch) * kBK;
            if (!A_MN) {
              tma_prefetch_2d(&tmA, kp, m0);
            } else {
#pragma unroll
              for (int c = 0; c < kBM / 64; ++c) tma_prefetch_2d(&tmA, m0 + c * 64, kp);
            }
            if (!B_MN) {
              tma_prefetch_2d(&tmB, kp, n0);
            } else {
#pragma unroll
              for (int c = 0; c < HB / 64; ++c) tma_prefetch_2d(&tmB, n0 + c * 64, kp);
            }
          }
          const uint32_t bar = mapa_u32(smem_u32(&full[stage]), 0);
          if (!A_MN) {
            tma_load_2d_pair(sA, &tmA, bar, kb * kBK, m0);
          } else {
#pragma unroll
            for (int c = 0; c < kBM / 64; ++c)
              tma_load_2d_pair(sA + c * (kBK * 128), &tmA, bar, m0 + c * 64, kb * kBK);
          }
          if (!B_MN) {
            tma_load_2d_pair(sB, &tmB, bar, kb * kBK, n0);
          } else {
#pragma unroll
            for (int c = 0; c < HB / 64; ++c)
              tma_load_2d_pair(sB + c * (kBK * 128), &tmB, bar, n0 + c * 64, kb * kBK);
          }
          if (++stage == S) { stage = 0; phase ^= 1; }
        }
      }
      if (TRACE) { tr[2] = stall; tr[3] = clock64(); }
    }
  } else if (warp == 1) {
    if (cta == 0 && elect_one()) {
      constexpr uint32_t idesc = umma_idesc_f16(Elem<T>::fmt, A_MN ? 1 : 0, B_MN ? 1 : 0, 2 * kBM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      long long stall_full = 0, stall_acc = 0;
      for (int tile = pair; tile < p.num_tiles && ok; tile += npairs, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        const long long t_a = TRACE ? clock64() : 0;
        ok = mbar_wait(&tempty[acc], acc_phase ^ 1, wctx, kErrWaitTmemEmpty);
        if (!ok) break;
        if (TRACE) stall_acc += clock64() - t_a;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          const long long t_w = TRACE ? clock64() : 0;
          ok = mbar_wait(&full[stage], phase, wctx, kErrWaitMma);
          if (!ok) break;
          if (TRACE) {
            const long long now = clock64();
            if (it == 0 && kb == 0) tr[4] = now;
            else stall_full += now - t_w;
          }
          tc_fence_after();
          const uint32_t a_base = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t b_base = a_base + Cfg::kABytes;
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t da = A_MN ? umma_desc_sw128(a_base + k * 2048, kBK * 128, 1024)
                                     : umma_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t db = B_MN ? umma_desc_sw128(b_base + k * 2048, kBK * 128, 1024)
                                     : umma_desc_sw128(b_base + k * 32, 16, 1024);
            umma_f16_pair(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty[stage], 3);
          if (++stage == S) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_pair(&tfull[acc], 3);
      }
      if (TRACE) { tr[5] = stall_full; tr[6] = stall_acc; tr[7] = clock64(); tr[8] = it; }
    }
  } else if (warp < 10) {
    const int quarter = warp & 3;      // TMEM lane quarter this warp may access
    const int half = (warp - 2) >> 2;  // which of the two warps of that quarter
    EpiStage es{epi_smem + (warp - 2) * kEpiBytesPerWarp, 0};
    int it = 0;
    bool ok = true;
    // AR: index (into this rank's owned tiles) of the next one this CTA reduces
    int next_owned = (AR && !ar.exchange) ? static_cast<int>(blockIdx.x) : 0;
    const int n_owned = !AR ? 0
                        : ar.exchange ? (p.num_tiles - pair + npairs - 1) / npairs
                                      : (num_m128 * ((p.N + BN - 1) / BN) - ar.rank + ar.tp - 1) / ar.tp;
    long long stall_epi = 0, cyc_ld = 0, cyc_rest = 0;
    long long cyc3[5] = {0, 0, 0, 0, 0};
    for (int tile = pair; tile < p.num_tiles && ok; tile += npairs, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      int m_idx, n_idx;
      pair_tile_coords(p, tile, m_idx, n_idx);
      // checked build: the tile order must stay inside the grid (the tile's own stores go through
      // the tensor map, which clips; the peer accesses below are guarded one by one)
      (void)TP_CHECK(m_idx >= 0 && m_idx < p.num_m_tiles && n_idx >= 0 && n_idx * BN < p.N, p.err,
                     kErrCheckTile);
      const int m0 = m_idx * (2 * kBM) + static_cast<int>(cta) * kBM;
      const int n0 = n_idx * BN;
      const long long t_e = TRACE ? clock64() : 0;
      ok = mbar_wait(&tfull[acc], acc_phase, wctx, kErrWaitEpilogue);
      if (!ok) break;
      if (TRACE && threadIdx.x == 64) {
        const long long now = clock64();
        stall_epi += now - t_e;
        if (it == 0) tr[9] = now;
        tr[10] = now;  // accumulator of the last tile became ready
      }
      tc_fence_after();
      const int row0 = m0 + quarter * 32;
      if (RS) {
        const int unit = m0 / kBM + n_idx * num_m128;   // 128-row block x column tile
        const int owner = min(row0 / ar.rows_per_rank, ar.tp - 1);
        const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
        const long long tile_elems = kBM * BN;
        const bool mine = row0 < p.M && owner == ar.rank;
        // checked build: the block's slot in the staging and flag arrays, and the owner's rank
        // (rows past M belong to no block: nothing of theirs is accessed)
        const bool slot_ok = row0 >= p.M ||
                             (TP_CHECK(unit >= 0 && unit < ar.max_tiles, p.err, kErrCheckStaging) &&
                              TP_CHECK(owner >= 0 && owner < ar.tp && ar.tp <= kMaxTp, p.err, kErrCheckPeer));
        // Hand this warp's part of the block to the publishing warp (which keeps at most two
        // blocks outstanding).  A warp that owns its rows has nothing to publish and says so
        // BEFORE it waits for its peers: their publishing warps wait for all eight epilogue warps
        // too, so waiting first would deadlock two ranks on a block that holds rows of both.
        auto pub_arrive = [&]() {
          if (it >= 2) {
            unsigned spins = 0;
            unsigned long long t0 = 0;
            while (*pub_done < it - 1 && !*abort_flag) {
              if ((++spins & 0xFF) == 0) {
                const unsigned long long now = globaltimer_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > g_wait_limit_ns) { report_timeout(wctx, kErrWaitEpilogue); break; }
              }
            }
          }
          mbar_arrive(&pub_full[it & 1]);
        };
        if (mine) {
          // rows of this rank: the other ranks' partials join the accumulator in the epilogue
          int got = 1;
          if (lane == 0) pub_arrive();
          if (lane == 0) {
            if (!slot_ok) got = 0;
            for (int src = 0; src < ar.tp && got; ++src)
              if (src != ar.rank)
                got = wait_flag(ar.flag_a[ar.rank] + static_cast<long long>(unit) * kMaxTp + src, ar_epoch,
                                wctx, kErrWaitPeer) ? 1 : 0;
          }
          got = __shfl_sync(0xffffffffu, got, 0);
          const T* part = static_cast<const T*>(ar.stage[ar.rank]) + stage_half + unit * tile_elems +
                          quarter * 1024 + lane * 32;
          const int nc = (min(BN, p.N - n0) + 31) / 32;
          epilogue_rows<T, OUT_F32, false>(p, &tmO, es, t_acc, nc, row0, n0, lane, half, 2, nullptr,
                                           got ? part : nullptr, ar.max_tiles * tile_elems, ar.tp, ar.rank);
        } else if (row0 < p.M) {
          // rows of another rank: 16-bit partial chunks into its staging buffer
          if (es.issued > 0) {          // the buffers may still be read by earlier tile stores
            if (lane == 0) bulk_wait_read<0>();
            __syncwarp();
          }
          T* dst = static_cast<T*>(ar.stage[owner]) + stage_half +
                   (static_cast<long long>(ar.rank) * ar.max_tiles + unit) * tile_elems + quarter * 1024;
#pragma unroll 1
          for (int c = half; c < BN / 32; c += 2) {
            uint32_t r[32];
            __syncwarp();
            tmem_ld_32x32(t_acc + c * 32, r);
            tmem_ld_wait();
            if (!slot_ok) continue;   // checked build: nothing is stored outside the staging buffer
            uint8_t* sb = es.buf + (c & 2 ? 2048 : 0);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 ov;
              ov.x = Elem<T>::pack2(__uint_as_float(r[g * 8 + 0]), __uint_as_float(r[g * 8 + 1]));
              ov.y = Elem<T>::pack2(__uint_as_float(r[g * 8 + 2]), __uint_as_float(r[g * 8 + 3]));
              ov.z = Elem<T>::pack2(__uint_as_float(r[g * 8 + 4]), __uint_as_float(r[g * 8 + 5]));
              ov.w = Elem<T>::pack2(__uint_as_float(r[g * 8 + 6]), __uint_as_float(r[g * 8 + 7]));
              *reinterpret_cast<uint4*>(sb + lane * 64 + ((g ^ ((lane >> 1) & 3)) << 4)) = ov;
            }
            __syncwarp();
            uint4* blk = reinterpret_cast<uint4*>(dst + c * 4096);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int piece = lane + 32 * k;
              const int rr = piece >> 2, part = piece & 3;
              blk[piece] = *reinterpret_cast<const uint4*>(sb + rr * 64 + ((part ^ ((rr >> 1) & 3)) << 4));
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive_cluster(mapa_u32(smem_u32(&tempty[acc]), 0));
          if (!mine) pub_arrive();
        }
        continue;
      }
      if (AR) {
        // phase A: this warp's chunks of the partial tile go to the owner's staging buffer
        const int m128 = m0 / kBM;
        const int ar_tile = m128 + n_idx * num_m128;
        // M may end inside the pair tile (warp-uniform); checked build: the tile's slot exists
        const bool in_range = m128 < num_m128 &&
                              TP_CHECK(ar_tile >= 0 && ar_tile < ar.max_tiles && ar.tp <= kMaxTp, p.err,
                                       kErrCheckStaging);
        const int owner = ar_tile % ar.tp;
        const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
        T* tile_dst = static_cast<T*>(ar.stage[owner]) +
                      (static_cast<long long>(ar.rank) * ar.max_tiles + ar_tile) * (kBM * BN);
#pragma unroll 1
        for (int c = half; c < BN / 32; c += 2) {
          uint32_t r[32];
          __syncwarp();
          tmem_ld_32x32(t_acc + c * 32, r);
          tmem_ld_wait();
          if (!in_range) continue;
          uint8_t* sb = es.buf + (es.issued & 1) * 2048;
          ++es.issued;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 ov;
            ov.x = Elem<T>::pack2(__uint_as_float(r[g * 8 + 0]), __uint_as_float(r[g * 8 + 1]));
            ov.y = Elem<T>::pack2(__uint_as_float(r[g * 8 + 2]), __uint_as_float(r[g * 8 + 3]));
            ov.z = Elem<T>::pack2(__uint_as_float(r[g * 8 + 4]), __uint_as_float(r[g * 8 + 5]));
            ov.w = Elem<T>::pack2(__uint_as_float(r[g * 8 + 6]), __uint_as_float(r[g * 8 + 7]));
            *reinterpret_cast<uint4*>(sb + lane * 64 + ((g ^ ((lane >> 1) & 3)) << 4)) = ov;
          }
          __syncwarp();
          // block (c, quarter): 2 KB contiguous at the owner; lane i copies 16-byte pieces
          // i, i + 32, i + 64, i + 96 (piece = row * 4 + part).  Exchange mode: to every rank.
          const long long blk_off = stage_half +
                                    (static_cast<long long>(ar.rank) * ar.max_tiles + ar_tile) * (kBM * BN) +
                                    (c * 4 + quarter) * 1024;
          uint4 pv[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int piece = lane + 32 * k;
            const int rr = piece >> 2, part = piece & 3;
            pv[k] = *reinterpret_cast<const uint4*>(sb + rr * 64 + ((part ^ ((rr >> 1) & 3)) << 4));
          }
          if (ar.exchange) {
            for (int dst = 0; dst < ar.tp; ++dst) {
              uint4* blk = reinterpret_cast<uint4*>(static_cast<T*>(ar.stage[dst]) + blk_off);
#pragma unroll
              for (int k = 0; k < 4; ++k) blk[lane + 32 * k] = pv[k];
            }
          } else {
            uint4* blk = reinterpret_cast<uint4*>(static_cast<T*>(ar.stage[owner]) + blk_off);
#pragma unroll
            for (int k = 0; k < 4; ++k) blk[lane + 32 * k] = pv[k];
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tempty[acc]), 0));
        // publish the tile once all eight warps have stored their blocks (named barrier 2); the
        // release store is cumulative over the writes ordered before it by the barrier
        asm volatile("bar.sync 2, 256;" ::: "memory");
        if (threadIdx.x == 64 && in_range) {
          if (ar.exchange) {
            for (int dst = 0; dst < ar.tp; ++dst)
              st_release_sys(ar.flag_a[dst] + static_cast<long long>(ar_tile) * kMaxTp + ar.rank, ar_epoch);
          } else {
            st_release_sys(ar.flag_a[owner] + static_cast<long long>(ar_tile) * kMaxTp + ar.rank, ar_epoch);
          }
        }
        // Phase B between tiles: while the tensor core works on the next tile, the epilogue
        // warps look (once, without waiting) whether a tile this CTA is to reduce has arrived
        // from every rank, and if so reduce it now.  Reduce-scatter mode: the next tile of this
        // rank's share; exchange mode: the oldest of this CTA's own tiles not yet reduced.
        if (next_owned < n_owned) {
          int otile;
          bool o_in_range = true;
          if (ar.exchange) {  // next_owned counts this CTA's own tiles
            const int t2 = pair + next_owned * npairs;
            const int o128 = (t2 % p.num_m_tiles) * 2 + static_cast<int>(cta);
            otile = o128 + (t2 / p.num_m_tiles) * num_m128;
            o_in_range = o128 < num_m128;
          } else {            // next_owned indexes the tiles this rank owns
            otile = next_owned * ar.tp + ar.rank;
          }
          o_in_range = o_in_range && TP_CHECK(otile >= 0 && otile < ar.max_tiles, p.err, kErrCheckStaging);
          if (threadIdx.x == 64) {
            bool ready = true;
            if (o_in_range)
              for (int src = 0; src < ar.tp; ++src)
                ready = ready &&
                        ld_acquire_sys(ar.flag_a[ar.rank] + static_cast<long long>(otile) * kMaxTp + src) >= ar_epoch;
            *s_ready = ready ? 1 : 0;
          }
          asm volatile("bar.sync 2, 256;" ::: "memory");
          if (*s_ready) {
            if (o_in_range) ar_reduce_tile<T, BN>(p, ar, otile, num_m128, threadIdx.x - 64, 256, ar.exchange != 0, stage_half);
            if (!ar.exchange) {
              asm volatile("bar.sync 2, 256;" ::: "memory");
              if (o_in_range && threadIdx.x >= 64 && threadIdx.x < 64 + ar.tp)
                st_release_sys(ar.flag_b[threadIdx.x - 64] + otile, ar_epoch);
            }
            next_owned += ar.exchange ? 1 : static_cast<int>(gridDim.x);
          }
        }
        continue;
      }
      if (row0 < p.M) {
        const int nc = (min(BN, p.N - n0) + 31) / 32;
        const long long t_l = TRACE ? clock64() : 0;
        epilogue_rows<T, OUT_F32, TRACE>(
            p, &tmO, es, tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN, nc, row0,
            n0, lane, half, 2, cyc3);
        if (TRACE) cyc_rest += clock64() - t_l;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tempty[acc]), 0));
    }
    if (TRACE && threadIdx.x == 64) { tr[11] = stall_epi; tr[12] = clock64(); tr[14] = cyc_ld; tr[15] = cyc_rest;
      tr[16] = cyc3[0]; tr[17] = cyc3[1]; tr[18] = cyc3[2]; tr[19] = cyc3[3]; tr[20] = cyc3[4]; }
    epi_drain(lane);  // the staging buffers must outlive the stores that read them
    if (AR && threadIdx.x == 64) {
      *s_next = next_owned;
    }
  }

  if (RS && warp == 10 && lane == 0) {
    // publishing warp: after all eight epilogue warps have stored their part of a 128-row block,
    // make the stores visible system-wide and raise the block's flag at every rank that owns rows
    // of it.  The release fence waits for the NVLink round trip; only this thread pays for it.
    int it = 0;
    bool ok = true;
    for (int tile = pair; tile < p.num_tiles && ok; tile += npairs, ++it) {
      int m_idx, n_idx;
      pair_tile_coords(p, tile, m_idx, n_idx);
      const int m0 = m_idx * (2 * kBM) + static_cast<int>(cta) * kBM;
      ok = mbar_wait(&pub_full[it & 1], (it >> 1) & 1, wctx, kErrWaitEpilogue);
      if (!ok) break;
      if (m0 < p.M) {
        const int unit = m0 / kBM + n_idx * num_m128;
        int last = -1;
        bool fenced = false;
        for (int q = 0; q < 4; ++q) {
          const int row0 = m0 + q * 32;
          if (row0 >= p.M) break;
          const int owner = min(row0 / ar.rows_per_rank, ar.tp - 1);
          if (owner == ar.rank || owner == last) continue;
          if (!TP_CHECK(unit >= 0 && unit < ar.max_tiles, p.err, kErrCheckStaging) ||
              !TP_CHECK(owner >= 0 && owner < ar.tp, p.err, kErrCheckPeer))
            continue;
          if (!fenced) {
            __threadfence_system();
            fenced = true;
          }
          asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(
                           ar.flag_a[owner] + static_cast<long long>(unit) * kMaxTp + ar.rank),
                       "r"(ar_epoch)
                       : "memory");
          last = owner;
        }
      }
      *pub_done = it + 1;
    }
  }

  if (AR) {
    __syncthreads();
    __shared__ int s_ok;
    // phase B, remainder: the tiles that were not reduced between this CTA's own tiles
    const int num_ar_tiles = num_m128 * ((p.N + BN - 1) / BN);
    const int nthreads = static_cast<int>(blockDim.x);
    if (ar.exchange) {
      const int n_mine = (p.num_tiles - pair + npairs - 1) / npairs;
      for (int seq = *s_next; seq < n_mine; ++seq) {
        const int t2 = pair + seq * npairs;
        const int o128 = (t2 % p.num_m_tiles) * 2 + static_cast<int>(cta);
        if (o128 >= num_m128) continue;  // uniform over the CTA
        const int tile = o128 + (t2 / p.num_m_tiles) * num_m128;
        if (!TP_CHECK(tile >= 0 && tile < ar.max_tiles, p.err, kErrCheckStaging)) continue;
        if (threadIdx.x == 0) {
          bool ok = true;
          for (int src = 0; src < ar.tp && ok; ++src)
            ok = wait_flag(ar.flag_a[ar.rank] + static_cast<long long>(tile) * kMaxTp + src, ar_epoch, wctx,
                           kErrWaitPeer);
          s_ok = ok ? 1 : 0;
        }
        __syncthreads();
        if (s_ok) ar_reduce_tile<T, BN>(p, ar, tile, num_m128, threadIdx.x, nthreads, true, stage_half);
        __syncthreads();
      }
    } else {
      const int n_owned = (num_ar_tiles - ar.rank + ar.tp - 1) / ar.tp;
      for (int j = *s_next; j < n_owned; j += gridDim.x) {
        const int tile = j * ar.tp + ar.rank;
        if (!TP_CHECK(tile >= 0 && tile < ar.max_tiles, p.err, kErrCheckStaging)) continue;
        if (threadIdx.x == 0) {
          bool ok = true;
          for (int src = 0; src < ar.tp && ok; ++src)
            ok = wait_flag(ar.flag_a[ar.rank] + static_cast<long long>(tile) * kMaxTp + src, ar_epoch, wctx,
                           kErrWaitPeer);
          s_ok = ok ? 1 : 0;
        }
        __syncthreads();
        if (s_ok) ar_reduce_tile<T, BN>(p, ar, tile, num_m128, threadIdx.x, nthreads, false, stage_half);
        __syncthreads();
        if (s_ok && threadIdx.x < ar.tp) st_release_sys(ar.flag_b[threadIdx.x] + tile, ar_epoch);
      }
      // phase C: every tile of the output must have arrived in this rank's memory
      for (int tile = blockIdx.x * nthreads + threadIdx.x; tile < num_ar_tiles; tile += gridDim.x * nthreads)
        if (TP_CHECK(tile < ar.max_tiles, p.err, kErrCheckStaging))
          wait_flag(ar.flag_b[ar.rank] + tile, ar_epoch, wctx, kErrWaitPeer);
    }
    __syncthreads();
  }

  // teardown: nobody leaves (or frees TMEM) while the peer may still read this CTA's shared
  // memory or signal its barriers.  On an aborted run give in-flight copies time to land first.
  __syncthreads();
  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  if (warp == 1) tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
  if (TRACE && threadIdx.x == 0) tr[13] = clock64();
}

static int max_pairs() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return num_sms() / 2;
  if (cached[dev] == 0) cached[dev] = num_sms() / 2;
  return cached[dev];
}

template <typename T, int BN, bool A_MN, bool B_MN, bool OUT_F32, bool TRACE = false, bool AR = false,
          bool RS = false>
static int launch_gemm_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmO,
                            const GemmParams& p, cudaStream_t stream, const ArParams* arp = nullptr) {
  using Cfg = PairCfg<BN>;
  auto kern = gemm_pair_kernel<T, BN, A_MN, B_MN, OUT_F32, TRACE, AR, RS>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) !=
        cudaSuccess)
      return kErrLaunch;
    configured = true;
  }
  ArParams ar;
  if (arp) ar = *arp;
  else { ar.tp = 0; ar.exchange = 0; ar.rows_per_rank = 0; }
  const int pairs = p.num_tiles < max_pairs() ? p.num_tiles : max_pairs();
  return launch_pdl(kern, dim3(2 * pairs), dim3(kPairThreads + (RS ? 32 : 0)), Cfg::kSmemBytes, stream, 2,
                    tmA, tmB, tmO, p, ar) == cudaSuccess
             ? kOk
             : kErrLaunch;
}

template <typename T, int BN>
static int dispatch_layout_pair(int a_mn, int b_mn, int out_f32, const CUtensorMap& tmA,
                                const CUtensorMap& tmB, const CUtensorMap& tmO, const GemmParams& p,
                                cudaStream_t s) {
  if (!a_mn && !b_mn && !out_f32) return launch_gemm_pair<T, BN, false, false, false>(tmA, tmB, tmO, p, s);
  if (!a_mn && b_mn && !out_f32) return launch_gemm_pair<T, BN, false, true, false>(tmA, tmB, tmO, p, s);
  if (a_mn && b_mn && out_f32) return launch_gemm_pair<T, BN, true, true, true>(tmA, tmB, tmO, p, s);
  return kErrBadArgument;
}

// Tile choice.  Codes: 64 / 128 / 256 = one CTA, 128 x BN tile; 512 = one CTA, 256 x 256;
// 1128 / 1256 = CTA pair, 256 x 128 / 256 x 256.  Relative time of one tile =
// (tile FLOPs per SM) / (fraction of the MMA rate the shared-memory feed sustains for that
// shape); total = waves x that.  Wave quantisation matters because M is only ~1024 rows per
// token slice.
static bool g_pair_default = true;
static int g_prefetch = 0;             // L2 prefetch distance of the CTA-pair kernel, in k-steps
static bool g_ar_exchange = false;     // one-hop exchange instead of reduce-scatter + all-gather

// Measured model of one launch, in kilo-cycles: waves x (main loop of one tile, proportional to
// K, + epilogue where it does not overlap the next tile) + exposed epilogue of the last tile.
// `loop` is per 2048 of K: the CTA-pair tiles run at 80-98 % of the MMA rate, the one-CTA tiles
// at 50-67 % (L2 -> shared-memory feed of one SM).
struct TileCand {
  int code, bm, bn;
  bool pair;
  float loop, epi_each, tail;
};
static const TileCand kTileCands[6] = {
    {1256, 256, 256, true, 16.7f, 0.0f, 8.5f}, {1128, 256, 128, true, 10.0f, 0.0f, 5.5f},
    {512, 256, 256, false, 36.0f, 18.0f, 0.0f}, {256, 128, 256, false, 24.7f, 0.0f, 10.0f},
    {128, 128, 128, false, 16.4f, 0.0f, 5.4f}, {64, 128, 64, false, 9.5f, 0.0f, 3.0f}};

static int pick_tile(int M, int N, int K, int forced, bool allow_256x256, bool allow_pair) {
  if (forced == 64 || forced == 128 || forced == 256) return forced;
  if (forced == 512) return allow_256x256 ? 512 : 256;
  if (forced == 1128 || forced == 1256) return allow_pair ? forced : forced - 1000;
  const int sms = num_sms();
  int best = 128;
  float best_t = 1e30f;
  for (const TileCand& c : kTileCands) {
    if (c.code == 512 && !allow_256x256) continue;
    if (c.pair && !(allow_pair && g_pair_default)) continue;
    const int tiles = ((M + c.bm - 1) / c.bm) * ((N + c.bn - 1) / c.bn);
    const int slots = c.pair ? sms / 2 : sms;
    const float waves = static_cast<float>((tiles + slots - 1) / slots);
    const float t = waves * (c.loop * static_cast<float>(K) / 2048.0f + c.epi_each) + c.tail;
    if (t < best_t) { best_t = t; best = c.code; }
  }
  return best;
}

}  // namespace tp

namespace tp {
// All-gather wait of a product whose A rows were pushed into this GPU's memory by the ranks of a
// tensor-parallel group (see GemmParams::ag_flags).
struct AgWait {
  const int* flags;
  const int* epoch_base;
  int epoch, rows_per_rank, rank;
};
}  // namespace tp

static int gemm_impl(int dtype, int a_mn, int b_mn, const void* A, long long lda, const void* B,
                     long long ldb, void* out, long long ldo, int out_f32, int accumulate, int M,
                     int N, int K, float alpha, const void* bias, const void* residual,
                     long long ldr, int act, void* aux_out, int dact, const void* aux_in,
                     long long ld_aux, int force_bn, int* err_flag, void* stream,
                     const tp::AgWait* ag) {
  using namespace tp;
  if (M <= 0 || N <= 0 || K <= 0) return kErrBadArgument;
  if ((N % 8) || (lda % 8) || (ldb % 8) || (ldo % (out_f32 ? 4 : 8))) return kErrBadArgument;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return kErrBadArgument;
  if (accumulate && !out_f32) return kErrBadArgument;
  const bool bf16 = dtype == 1;
  const bool common_layout = (!a_mn && !out_f32) || (a_mn && b_mn && out_f32);
  // only the three layouts of a Linear layer's forward / dgrad / wgrad products have the
  // 256-row tiles instantiated
  int tile_code = pick_tile(M, N, K, force_bn, common_layout, common_layout);
  if (ag) {
    // the wait lives in the CTA-pair kernel's producer
    if (a_mn || !common_layout || ag->rows_per_rank <= 0) return kErrBadArgument;
    if (tile_code < 1000) tile_code = (N % 256 == 0 && N >= 2048) ? 1256 : 1128;
  }
  const bool pair = tile_code > 1000;
  const int BN = pair ? tile_code - 1000 : (tile_code == 512 ? 256 : tile_code);
  const int BM = (pair || tile_code == 512) ? 256 : kBM;   // rows of one output tile
  const int box_m = pair ? kBM : BM;                       // rows of A one CTA loads
  const int box_n = pair ? BN / 2 : BN;                    // rows of B one CTA loads
  CUtensorMap tmA, tmB;
  bool ok;
  if (!a_mn) ok = make_tmap_2d(&tmA, A, K, M, lda, kBK, box_m, bf16);
  else ok = make_tmap_2d(&tmA, A, M, K, lda, 64, kBK, bf16);
  if (!ok) return kErrDriver;
  if (!b_mn) ok = make_tmap_2d(&tmB, B, K, N, ldb, kBK, box_n, bf16);
  else ok = make_tmap_2d(&tmB, B, N, K, ldb, 64, kBK, bf16);
  if (!ok) return kErrDriver;
  CUtensorMap tmO;
  if (!make_tmap_out(&tmO, out, N, M, ldo, out_f32 != 0, bf16)) return kErrDriver;
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.num_m_tiles = (M + BM - 1) / BM;
  p.num_n_tiles = (N + BN - 1) / BN;
  p.num_tiles = p.num_m_tiles * p.num_n_tiles;
  p.m_major = 0; p.m_first = 0; p.order_split = 1; p.order_group = 1; p.order_first_only = 0; p.order_pipelined = 0;
  p.ag_flags = nullptr; p.ag_epoch_base = nullptr; p.ag_epoch = 0; p.ag_rows = 1; p.ag_rank = 0;
  if (ag) {
    // the first wave of tiles takes row blocks of this rank only: their operands are local
    // while the peers' rows are still arriving; later tiles use the ordinary order
    apply_tile_order(p, ag_tile_order(p.num_m_tiles, p.num_n_tiles, BM, ag->rank, ag->rows_per_rank,
                                      max_pairs()));
    p.ag_flags = ag->flags; p.ag_epoch_base = ag->epoch_base; p.ag_epoch = ag->epoch;
    p.ag_rows = ag->rows_per_rank; p.ag_rank = ag->rank;
  }
  p.out = out; p.ldo = ldo;
  p.bias = bias; p.residual = residual; p.ldr = ldr;
  p.aux_out = aux_out; p.aux_in = aux_in; p.ld_aux = ld_aux;
  p.alpha = alpha; p.act = act; p.dact = dact; p.accumulate = accumulate;
  p.err = err_flag;
  p.trace = nullptr;
  p.prefetch = g_prefetch;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define TP_DISPATCH(T)                                                                   \
  (pair ? (BN == 256 ? dispatch_layout_pair<T, 256>(a_mn, b_mn, out_f32, tmA, tmB, tmO, p, s)  \
                     : dispatch_layout_pair<T, 128>(a_mn, b_mn, out_f32, tmA, tmB, tmO, p, s)) \
   : tile_code == 512 ? dispatch_layout<T, 256, 2>(a_mn, b_mn, out_f32, tmA, tmB, tmO, p, s)  \
   : BN == 256 ? dispatch_layout<T, 256>(a_mn, b_mn, out_f32, tmA, tmB, tmO, p, s)            \
   : BN == 128 ? dispatch_layout<T, 128>(a_mn, b_mn, out_f32, tmA, tmB, tmO, p, s)            \
               : dispatch_layout<T, 64>(a_mn, b_mn, out_f32, tmA, tmB, tmO, p, s))
  return bf16 ? TP_DISPATCH(__nv_bfloat16) : TP_DISPATCH(__half);
#undef TP_DISPATCH
}

extern "C" int tp_gemm(int dtype, int a_mn, int b_mn, const void* A, long long lda, const void* B,
                       long long ldb, void* out, long long ldo, int out_f32, int accumulate, int M,
                       int N, int K, float alpha, const void* bias, const void* residual,
                       long long ldr, int act, void* aux_out, int dact, const void* aux_in,
                       long long ld_aux, int force_bn, int* err_flag, void* stream) {
  return gemm_impl(dtype, a_mn, b_mn, A, lda, B, ldb, out, ldo, out_f32, accumulate, M, N, K, alpha,
                   bias, residual, ldr, act, aux_out, dact, aux_in, ld_aux, force_bn, err_flag, stream,
                   nullptr);
}

// All-gather -> GEMM: the same product as tp_gemm for A stored [M][K] whose rows
// [s * rows_per_rank, (s + 1) * rows_per_rank) were written into this GPU's memory by rank s of a
// tensor-parallel group (peer stores of the producing kernel, e.g. tp_layernorm_fwd_push).  The
// kernel starts with the row blocks of rank `rank` and, before it loads rows of another rank s,
// waits (bounded) until ag_flags[s] >= ag_epoch + *ag_epoch_base; it reads its own memory only.
extern "C" int tp_gemm_ag(int dtype, int b_mn, const void* A, long long lda, const void* B,
                          long long ldb, void* out, long long ldo, int M, int N, int K,
                          const void* bias, int act, void* aux_out, int dact, const void* aux_in,
                          long long ld_aux, const int* ag_flags, const int* ag_epoch_base, int ag_epoch,
                          int rows_per_rank, int rank, int* err_flag, void* stream) {
  tp::AgWait ag{ag_flags, ag_epoch_base, ag_epoch, rows_per_rank, rank};
  return gemm_impl(dtype, 0, b_mn, A, lda, B, ldb, out, ldo, 0, 0, M, N, K, 1.0f, bias, nullptr, 0, act,
                   aux_out, dact, aux_in, ld_aux, 0, err_flag, stream, ag_flags ? &ag : nullptr);
}

// Fused GEMM + tensor-parallel all-reduce (see the file comment).  `out_ptrs[r]` is the address
// of the output matrix in rank r's memory (peer-mapped), `stage_ptrs` / `flag_*_ptrs` the
// staging and flag arrays of every rank.  All-reduce tiles are 128 x 128; the product runs on
// 256 x 128 CTA-pair tiles unless tp_gemm_set_pair_default(0) selected the one-CTA kernel.  Every rank of the group must
// make the same call with the same epoch = `epoch` + *`epoch_base`; the sum must grow from call
// to call (epoch = index of the call within a step, *epoch_base advanced per step on the device).
extern "C" int tp_gemm_ar(int dtype, int b_mn, const void* A, long long lda, const void* B,
                          long long ldb, long long ldo, int M, int N, int K, const void* bias,
                          const void* residual, long long ldr, int tp, int rank, int epoch,
                          const int* epoch_base, int max_tiles, void* const* stage_ptrs, int* const* flag_a_ptrs,
                          int* const* flag_b_ptrs, void* const* out_ptrs, int* err_flag,
                          void* stream) {
  using namespace tp;
  if (M <= 0 || N <= 0 || K <= 0 || tp < 2 || tp > kMaxTp || rank < 0 || rank >= tp)
    return kErrBadArgument;
  if ((N % 8) || (lda % 8) || (ldb % 8) || (ldo % 8)) return kErrBadArgument;
  constexpr int BN = 128;
  const bool bf16 = dtype == 1;
  const bool pair = g_pair_default;  // 256 x 128 CTA-pair tiles; all-reduce tiles stay 128 x 128
  const int BM = pair ? 2 * kBM : kBM;
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.num_m_tiles = (M + BM - 1) / BM;
  p.num_n_tiles = (N + BN - 1) / BN;
  p.num_tiles = p.num_m_tiles * p.num_n_tiles;
  p.m_major = 0; p.m_first = 0; p.order_split = 1; p.order_group = 1; p.order_first_only = 0; p.order_pipelined = 0;
  p.ag_flags = nullptr; p.ag_epoch_base = nullptr; p.ag_epoch = 0; p.ag_rows = 1; p.ag_rank = 0;
  if (((M + kBM - 1) / kBM) * ((N + BN - 1) / BN) > max_tiles) return kErrTooLarge;
  CUtensorMap tmA, tmB;
  if (!make_tmap_2d(&tmA, A, K, M, lda, kBK, kBM, bf16)) return kErrDriver;
  if (!(b_mn ? make_tmap_2d(&tmB, B, N, K, ldb, 64, kBK, bf16)
             : make_tmap_2d(&tmB, B, K, N, ldb, kBK, pair ? BN / 2 : BN, bf16)))
    return kErrDriver;
  p.out = out_ptrs[rank]; p.ldo = ldo;
  p.bias = bias; p.residual = residual; p.ldr = ldr;
  p.aux_out = nullptr; p.aux_in = nullptr; p.ld_aux = 0;
  p.alpha = 1.0f; p.act = 0; p.dact = 0; p.accumulate = 0;
  p.err = err_flag;
  p.trace = nullptr;
  p.prefetch = g_prefetch;
  ArParams ar;
  ar.tp = tp; ar.rank = rank; ar.epoch = epoch; ar.epoch_base = epoch_base; ar.max_tiles = max_tiles;
  ar.exchange = (g_pair_default && g_ar_exchange) ? 1 : 0;
  ar.rows_per_rank = 0;
  for (int i = 0; i < kMaxTp; ++i) {
    ar.stage[i] = i < tp ? stage_ptrs[i] : nullptr;
    ar.flag_a[i] = i < tp ? flag_a_ptrs[i] : nullptr;
    ar.flag_b[i] = i < tp ? flag_b_ptrs[i] : nullptr;
    ar.out[i] = i < tp ? out_ptrs[i] : nullptr;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const CUtensorMap& tmO = tmA;  // the fused all-reduce epilogue stores through peer pointers
  if (pair) {
    if (bf16)
      return b_mn ? launch_gemm_pair<__nv_bfloat16, BN, false, true, false, false, true>(tmA, tmB, tmO, p, s, &ar)
                  : launch_gemm_pair<__nv_bfloat16, BN, false, false, false, false, true>(tmA, tmB, tmO, p, s, &ar);
    return b_mn ? launch_gemm_pair<__half, BN, false, true, false, false, true>(tmA, tmB, tmO, p, s, &ar)
                : launch_gemm_pair<__half, BN, false, false, false, false, true>(tmA, tmB, tmO, p, s, &ar);
  }
  if (bf16)
    return b_mn ? launch_gemm<__nv_bfloat16, BN, false, true, false, true>(tmA, tmB, tmO, p, s, &ar)
                : launch_gemm<__nv_bfloat16, BN, false, false, false, true>(tmA, tmB, tmO, p, s, &ar);
  return b_mn ? launch_gemm<__half, BN, false, true, false, true>(tmA, tmB, tmO, p, s, &ar)
              : launch_gemm<__half, BN, false, false, false, true>(tmA, tmB, tmO, p, s, &ar);
}

// Fused GEMM + tensor-parallel reduce-scatter over the rows (CTA-pair kernel, 256 x 128 tiles):
// every rank computes its K shard of out = A * B^T (or A * B for b_mn) for all M rows; rank s ends
// with rows [s * rows_per_rank, (s + 1) * rows_per_rank) of the sum, plus bias and residual, in
// its own `out` (same row indices as the full matrix; other rows are not written).
// rows_per_rank must be a multiple of 32; tiles are visited so that this rank's rows come last.
// `stage_ptrs` / `flag_ptrs` are the staging and flag arrays of every rank as for tp_gemm_ar (two
// staging halves, alternating with the call counter); epoch rules as for tp_gemm_ar.
extern "C" int tp_gemm_rs(int dtype, int b_mn, const void* A, long long lda, const void* B,
                          long long ldb, void* out, long long ldo, int M, int N, int K,
                          const void* bias, const void* residual, long long ldr, int tp, int rank,
                          int rows_per_rank, int epoch, const int* epoch_base, int max_tiles,
                          void* const* stage_ptrs, int* const* flag_ptrs, int* err_flag, void* stream) {
  using namespace tp;
  if (M <= 0 || N <= 0 || K <= 0 || tp < 2 || tp > kMaxTp || rank < 0 || rank >= tp)
    return kErrBadArgument;
  if ((N % 8) || (lda % 8) || (ldb % 8) || (ldo % 8) || rows_per_rank <= 0 || (rows_per_rank % 32))
    return kErrBadArgument;
  if (static_cast<long long>(rows_per_rank) * tp < M) return kErrBadArgument;
  constexpr int BN = 128;
  const bool bf16 = dtype == 1;
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.num_m_tiles = (M + 2 * kBM - 1) / (2 * kBM);
  p.num_n_tiles = (N + BN - 1) / BN;
  p.num_tiles = p.num_m_tiles * p.num_n_tiles;
  if (((M + kBM - 1) / kBM) * p.num_n_tiles > max_tiles) return kErrTooLarge;
  // The row blocks of the other ranks first (starting after this rank's rows), this rank's own
  // row blocks last (tile_order.h).
  apply_tile_order(p, rs_tile_order(M, N, K, p.num_m_tiles, p.num_n_tiles, 2 * kBM, rank, rows_per_rank,
                                    max_pairs()));
  p.ag_flags = nullptr; p.ag_epoch_base = nullptr; p.ag_epoch = 0; p.ag_rows = 1; p.ag_rank = 0;
  CUtensorMap tmA, tmB, tmO;
  if (!make_tmap_2d(&tmA, A, K, M, lda, kBK, kBM, bf16)) return kErrDriver;
  if (!(b_mn ? make_tmap_2d(&tmB, B, N, K, ldb, 64, kBK, bf16)
             : make_tmap_2d(&tmB, B, K, N, ldb, kBK, BN / 2, bf16)))
    return kErrDriver;
  if (!make_tmap_out(&tmO, out, N, M, ldo, false, bf16)) return kErrDriver;
  p.out = out; p.ldo = ldo;
  p.bias = bias; p.residual = residual; p.ldr = ldr;
  p.aux_out = nullptr; p.aux_in = nullptr; p.ld_aux = 0;
  p.alpha = 1.0f; p.act = 0; p.dact = 0; p.accumulate = 0;
  p.err = err_flag;
  p.trace = nullptr;
  p.prefetch = g_prefetch;
  ArParams ar;
  ar.tp = tp; ar.rank = rank; ar.epoch = epoch; ar.epoch_base = epoch_base; ar.max_tiles = max_tiles;
  ar.exchange = 0; ar.rows_per_rank = rows_per_rank;
  for (int i = 0; i < kMaxTp; ++i) {
    ar.stage[i] = i < tp ? stage_ptrs[i] : nullptr;
    ar.flag_a[i] = i < tp ? flag_ptrs[i] : nullptr;
    ar.flag_b[i] = nullptr;
    ar.out[i] = nullptr;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (bf16)
    return b_mn ? launch_gemm_pair<__nv_bfloat16, BN, false, true, false, false, false, true>(tmA, tmB, tmO, p, s, &ar)
                : launch_gemm_pair<__nv_bfloat16, BN, false, false, false, false, false, true>(tmA, tmB, tmO, p, s, &ar);
  return b_mn ? launch_gemm_pair<__half, BN, false, true, false, false, false, true>(tmA, tmB, tmO, p, s, &ar)
              : launch_gemm_pair<__half, BN, false, false, false, false, false, true>(tmA, tmB, tmO, p, s, &ar);
}

TP_DEFINE_WAIT_LIMIT_SETTER(tp_set_wait_limit_ns_gemm)

namespace tp {
__global__ void advance_counter_kernel(int* counter, int inc) { *counter += inc; }
}  // namespace tp

// Phase trace of the CTA-pair kernel (fp16, out = A[M][K] * B[N][K]^T, no epilogue operands).
// `trace` receives 24 int64 slots per CTA (2 * min(tiles, SMs / 2) CTAs), SM clock cycles:
//   0 kernel entry, 1 set-up done (barriers, TMEM, cluster sync), 2 producer: cycles spent
//   waiting for free ring slots, 3 producer: last load issued, 4 MMA thread: first operands
//   arrived, 5 MMA thread: cycles waiting for operands (after the first), 6 MMA thread: cycles
//   waiting for a free accumulator, 7 MMA thread: last MMA issued, 8 tiles done, 9 epilogue:
//   first accumulator ready, 10 epilogue: last accumulator ready, 11 epilogue: cycles waiting
//   for accumulators, 12 epilogue: last store issued, 13 kernel exit, 14 epilogue: cycles in TMEM
//   loads, 15 epilogue: cycles in the math and stores of the chunks, split into 16 waiting for a
//   free staging buffer, 17 math and shared-memory writes, 18 proxy fence and store issue; first
//   chunk of every tile: 19 TMEM load issue until its wait returns, 20 until a loaded register reads.  Slots 4-8 are written by
//   the leader CTA of each pair only.
extern "C" int tp_gemm_trace(int bn, const void* A, long long lda, const void* B, long long ldb,
                             void* out, long long ldo, int M, int N, int K, long long* trace,
                             int* err_flag, void* stream) {
  using namespace tp;
  if (M <= 0 || N <= 0 || K <= 0 || (bn != 128 && bn != 256) || !trace) return kErrBadArgument;
  if ((N % 8) || (lda % 8) || (ldb % 8) || (ldo % 8)) return kErrBadArgument;
  CUtensorMap tmA, tmB;
  if (!make_tmap_2d(&tmA, A, K, M, lda, kBK, kBM, false)) return kErrDriver;
  if (!make_tmap_2d(&tmB, B, K, N, ldb, kBK, bn / 2, false)) return kErrDriver;
  CUtensorMap tmO;
  if (!make_tmap_out(&tmO, out, N, M, ldo, false, false)) return kErrDriver;
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.num_m_tiles = (M + 2 * kBM - 1) / (2 * kBM);
  p.num_n_tiles = (N + bn - 1) / bn;
  p.num_tiles = p.num_m_tiles * p.num_n_tiles;
  p.m_major = 0; p.m_first = 0; p.order_split = 1; p.order_group = 1; p.order_first_only = 0; p.order_pipelined = 0;
  p.ag_flags = nullptr; p.ag_epoch_base = nullptr; p.ag_epoch = 0; p.ag_rows = 1; p.ag_rank = 0;
  p.out = out; p.ldo = ldo;
  p.bias = nullptr; p.residual = nullptr; p.ldr = 0;
  p.aux_out = nullptr; p.aux_in = nullptr; p.ld_aux = 0;
  p.alpha = 1.0f; p.act = 0; p.dact = 0; p.accumulate = 0;
  p.err = err_flag;
  p.trace = trace;
  p.prefetch = g_prefetch;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return bn == 256 ? launch_gemm_pair<__half, 256, false, false, false, true>(tmA, tmB, tmO, p, s)
                   : launch_gemm_pair<__half, 128, false, false, false, true>(tmA, tmB, tmO, p, s);
}

// Fused all-reduce, CTA-pair kernel.  exchange = 1: every rank sends each partial tile to every
// rank and reduces all tiles itself (one NVLink hop, (tp - 1) x the bytes); 0 (default):
// reduce-scatter to an owner rank, then all-gather (two hops).  On two B200s the one-hop form
// measured slower (86 vs 72 us for 1024 x 5120 x 2560).
extern "C" void tp_gemm_ar_set_exchange(int enabled) { tp::g_ar_exchange = enabled != 0; }

// L2 prefetch distance (in 64-element k-steps) of the CTA-pair kernel's producer; 0 switches it off.
extern "C" void tp_gemm_set_prefetch(int k_steps) { tp::g_prefetch = k_steps < 0 ? 0 : k_steps; }

// Process-wide switch for the automatic tile choice: 0 keeps every GEMM on single-CTA tiles.
extern "C" void tp_gemm_set_pair_default(int enabled) { tp::g_pair_default = enabled != 0; }

extern "C" int tp_advance_counter(int* counter, int inc, void* stream) {
  tp::advance_counter_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(counter, inc);
  return cudaGetLastError() == cudaSuccess ? tp::kOk : tp::kErrLaunch;
}
