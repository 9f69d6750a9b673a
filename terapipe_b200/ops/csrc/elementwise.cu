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

template <typename T> __device__ __forceinline__ void load8(const T* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = Elem<T>::unpack2(w[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float (&f)[8]) {
  uint4 u;
  u.x = Elem<T>::pack2(f[0], f[1]);
  u.y = Elem<T>::pack2(f[2], f[3]);
  u.z = Elem<T>::pack2(f[4], f[5]);
  u.w = Elem<T>::pack2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// ------------------------------------------------------------------ LayerNorm forward
// y = (x - mean) * rstd * gamma + beta, one CTA per row; each thread keeps NV vectors of 8.
template <typename T, int NV>
__global__ void __launch_bounds__(NV == 1 ? 1024 : 768) layernorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gamma,
                                     const T* __restrict__ beta, T* __restrict__ y,
                                     float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                     int rows, int H, float eps) {
  __shared__ float red[33];
  const long long row = blockIdx.x;
  const T* xr = x + row * H;
  float v[NV][8];
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = (threadIdx.x + i * blockDim.x) * 8;
    if (col < H) {
      load8(xr + col, v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += v[i][j];
    }
  }
  const float mean = block_sum(s, red) / H;
  float q = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = (threadIdx.x + i * blockDim.x) * 8;
    if (col < H) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = v[i][j] - mean;
        q += d * d;
      }
    }
  }
  const float rstd = rsqrtf(block_sum(q, red) / H + eps);
  if (threadIdx.x == 0) {
    mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = (threadIdx.x + i * blockDim.x) * 8;
    if (col < H) {
      float g[8], b[8], o[8];
      load8(gamma + col, g);
      load8(beta + col, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mean) * rstd * g[j] + b[j];
      store8(y + row * H + col, o);
    }
  }
}

// ------------------------------------------------------------------ LayerNorm backward
// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)) (+ dres), g = dy * gamma.
// Persistent CTAs stride over rows and keep per-column partial sums of dgamma = sum dy*xhat
// and dbeta = sum dy in registers; partials go to `scratch[gridDim.x][2][H]` and a second
// kernel folds them into the fp32 gradient accumulators.
template <typename T, int NV, bool SMEM_PART>
__global__ void __launch_bounds__(NV == 1 ? 1024 : 768) layernorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                     const float* __restrict__ mean, const float* __restrict__ rstd,
                                     const T* __restrict__ gamma, const T* __restrict__ dres,
                                     T* __restrict__ dx, float* __restrict__ scratch, int rows,
                                     int H) {
  // For wide rows the per-column partial sums live in shared memory (each thread touches only
  // its own columns, so no synchronisation is needed); otherwise in registers.
  extern __shared__ float part_smem[];
  __shared__ float red[33];
  constexpr int NP = SMEM_PART ? 1 : NV;
  float pg[NP][8], pb[NP][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = (threadIdx.x + i * blockDim.x) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (SMEM_PART) {
        if (col < H) { part_smem[col + j] = 0.0f; part_smem[H + col + j] = 0.0f; }
      } else {
        pg[i % NP][j] = 0.0f;
        pb[i % NP][j] = 0.0f;
      }
    }
  }
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float mu = mean[row], rs = rstd[row];
    float xh[NV][8], g[NV][8];
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int col = (threadIdx.x + i * blockDim.x) * 8;
      if (col < H) {
        float xv[8], dyv[8], gam[8];
        load8(x + row * H + col, xv);
        load8(dy + row * H + col, dyv);
        load8(gamma + col, gam);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xv[j] - mu) * rs;
          g[i][j] = dyv[j] * gam[j];
          s1 += g[i][j];
          s2 += g[i][j] * xh[i][j];
          if (SMEM_PART) {
            part_smem[col + j] += dyv[j] * xh[i][j];
            part_smem[H + col + j] += dyv[j];
          } else {
            pg[i % NP][j] += dyv[j] * xh[i][j];
            pb[i % NP][j] += dyv[j];
          }
        }
      }
    }
    const float m1 = block_sum(s1, red) / H;
    const float m2 = block_sum(s2, red) / H;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int col = (threadIdx.x + i * blockDim.x) * 8;
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
        store8(dx + row * H + col, o);
      }
    }
  }
  float* sg = scratch + static_cast<long long>(blockIdx.x) * 2 * H;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = (threadIdx.x + i * blockDim.x) * 8;
    if (col < H) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        sg[col + j] = SMEM_PART ? part_smem[col + j] : pg[i % NP][j];
        sg[H + col + j] = SMEM_PART ? part_smem[H + col + j] : pb[i % NP][j];
      }
    }
  }
}

// dgamma[c] += sum_p scratch[p][0][c]; dbeta[c] += sum_p scratch[p][1][c]
__global__ void layernorm_bwd_reduce_kernel(const float* __restrict__ scratch, int parts, int H,
                                            float* __restrict__ dgamma, float* __restrict__ dbeta) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= 2 * H) return;
  float s = 0.0f;
  for (int p = 0; p < parts; ++p) s += scratch[static_cast<long long>(p) * 2 * H + c];
  if (c < H) dgamma[c] += s;
  else dbeta[c - H] += s;
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

static inline int ln_threads(int H, int nv) {
  int t = (H / 8 + nv - 1) / nv;
  t = (t + 31) / 32 * 32;
  return t;
}

extern "C" int tp_layernorm_fwd(int dtype, const void* x, const void* gamma, const void* beta,
                                void* y, float* mean, float* rstd, int rows, int H, float eps,
                                void* stream) {
  if (rows <= 0) return kOk;
  if (H % 8 || H > 12288) return kErrBadArgument;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int nv = H > 8192 ? 2 : 1;
  const int threads = ln_threads(H, nv);
#define LN_FWD(T, NV)                                                                         \
  layernorm_fwd_kernel<T, NV><<<rows, threads, 0, s>>>(                                       \
      static_cast<const T*>(x), static_cast<const T*>(gamma), static_cast<const T*>(beta),    \
      static_cast<T*>(y), mean, rstd, rows, H, eps)
  if (dtype == 1) { if (nv == 1) LN_FWD(__nv_bfloat16, 1); else LN_FWD(__nv_bfloat16, 2); }
  else { if (nv == 1) LN_FWD(__half, 1); else LN_FWD(__half, 2); }
#undef LN_FWD
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}

// Number of row-partial slots the backward writes; scratch must hold parts * 2 * H floats.
extern "C" int tp_layernorm_bwd_parts(int rows) {
  const int cap = 2 * num_sms();
  return rows < cap ? rows : cap;
}

namespace tp {
static int layernorm_bwd_launch(int dtype, const void* dy, const void* x, const float* mean,
                                const float* rstd, const void* gamma, const void* dres, void* dx,
                                float* dgamma, float* dbeta, float* scratch, int rows, int H,
                                cudaStream_t s) {
  if (rows <= 0) return kOk;
  if (H % 8 || H > 12288) return kErrBadArgument;
  const int nv = H > 8192 ? 2 : 1;
  const int threads = ln_threads(H, nv);
  const int parts = tp_layernorm_bwd_parts(rows);
#define LN_BWD(T, NV, SP)                                                                      \
  layernorm_bwd_kernel<T, NV, SP><<<parts, threads, (SP) ? 2 * H * sizeof(float) : 0, s>>>(    \
      static_cast<const T*>(dy), static_cast<const T*>(x), mean, rstd,                         \
      static_cast<const T*>(gamma), static_cast<const T*>(dres), static_cast<T*>(dx), scratch, \
      rows, H)
  if (nv == 2) {
    static bool attr_set = false;
    if (!attr_set) {
      cudaFuncSetAttribute(layernorm_bwd_kernel<__half, 2, true>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * 16384 * 4);
      cudaFuncSetAttribute(layernorm_bwd_kernel<__nv_bfloat16, 2, true>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * 16384 * 4);
      attr_set = true;
    }
  }
  if (dtype == 1) { if (nv == 1) LN_BWD(__nv_bfloat16, 1, false); else LN_BWD(__nv_bfloat16, 2, true); }
  else { if (nv == 1) LN_BWD(__half, 1, false); else LN_BWD(__half, 2, true); }
#undef LN_BWD
  layernorm_bwd_reduce_kernel<<<(2 * H + 255) / 256, 256, 0, s>>>(scratch, parts, H, dgamma, dbeta);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch;
}
}  // namespace tp

extern "C" int tp_layernorm_bwd(int dtype, const void* dy, const void* x, const float* mean,
                                const float* rstd, const void* gamma, const void* dres, void* dx,
                                float* dgamma, float* dbeta, float* scratch, int rows, int H,
                                void* stream) {
  return layernorm_bwd_launch(dtype, dy, x, mean, rstd, gamma, dres, dx, dgamma, dbeta, scratch,
                              rows, H, static_cast<cudaStream_t>(stream));
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
