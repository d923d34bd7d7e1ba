// Small operators around the mixers and feed-forwards of the hybrid families, each in 16- and 32-bit:
// an embedding that adds a sinusoidal position vector, the cast that joins two fp32 streams into one
// GEMM operand, plain (ungated) activations, an RMS norm that writes its rows into a cache pool, a
// per-head sigmoid gate, and an in-place scale of fp32 logits.  They follow hybrid_ops.cu's
// conventions (C ABI, no allocation, no sync); the reference has no model that needs them.
#include "common.cuh"
#include "ptx.cuh"

namespace spd {

constexpr int kLayThreads = 256;

// x[row, 2i] = table[id, 2i] + sin(p f_i), x[row, 2i+1] = table[id, 2i+1] + cos(p f_i), with f_i given as
// the sum of two floats (hi + lo, lo the rounding residue of the float64 frequency): the angle p f_i is
// formed as a product without rounding (fma residue) so that it is right to fp32 at any position.
template <typename T>
__global__ void __launch_bounds__(kLayThreads)
embed_sincos_kernel(float* __restrict__ x, const T* __restrict__ table, const int64_t* __restrict__ idx,
                    const int64_t* __restrict__ positions, const float* __restrict__ freq_hi,
                    const float* __restrict__ freq_lo, int64_t dim, int64_t table_rows) {
  griddep_wait();
  griddep_launch_dependents();
  const int64_t row = blockIdx.x;
  int64_t id = idx[row];
  id = id < 0 ? 0 : (id >= table_rows ? table_rows - 1 : id);
  const float p = (float)positions[row];  // exact below 2^24
  for (int64_t i = threadIdx.x; 2 * i < dim; i += kLayThreads) {
    const float a = p * freq_hi[i];
    const float rest = fmaf(p, freq_hi[i], -a) + p * freq_lo[i];  // p f - a: the product's rounding residue
    float sn, cs, sr, cr;
    sincosf(a, &sn, &cs);
    sincosf(rest, &sr, &cr);  // |rest| is a fraction of a radian even at a million positions
    const float s2 = fmaf(sn, cr, cs * sr), c2 = fmaf(cs, cr, -sn * sr);  // sin(a + rest), cos(a + rest)
    x[row * dim + 2 * i] = to_f32<T>(table[id * dim + 2 * i]) + s2;
    if (2 * i + 1 < dim) x[row * dim + 2 * i + 1] = to_f32<T>(table[id * dim + 2 * i + 1]) + c2;
  }
}

// out[row] = [a[row] | b[row]] in T (one operand of a GEMM over two fp32 streams)
template <typename T>
__global__ void __launch_bounds__(kLayThreads)
cast_concat_kernel(T* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b, int64_t dim) {
  griddep_wait();
  griddep_launch_dependents();
  const int64_t row = blockIdx.x;
  for (int64_t i = threadIdx.x; i < dim; i += kLayThreads) {
    out[row * 2 * dim + i] = from_f32<T>(a[row * dim + i]);
    out[row * 2 * dim + dim + i] = from_f32<T>(b[row * dim + i]);
  }
}

__device__ __forceinline__ float act_apply(float z, int act) {
  switch (act) {
    case 0: return z / (1.0f + expf(-z));                                                           // silu
    case 1: return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));   // gelu (tanh form)
    case 2: { const float r = fmaxf(z, 0.f); return r * r; }                                        // relu squared
    case 3: return tanhf(z);
    default: return fmaxf(z, 0.f);                                                                  // relu
  }
}

// vector form: cols and the row stride multiples of the vector width, 16-byte aligned pointers
template <typename T>
__global__ void __launch_bounds__(kLayThreads)
activation_vec_kernel(T* __restrict__ out, const T* __restrict__ x, int64_t rows, int64_t cols, int64_t x_stride,
                      int act) {
  griddep_wait();
  griddep_launch_dependents();
  constexpr int N = Vec16<T>::kN;
  const int64_t per_row = cols / N, n = rows * per_row;
  for (int64_t i = blockIdx.x * (int64_t)kLayThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kLayThreads) {
    const int64_t r = i / per_row, c = (i - r * per_row) * N;
    const Vec16<T> v = ldv(x + r * x_stride + c);
    Vec16<T> o;
#pragma unroll
    for (int k = 0; k < N; ++k) o.e()[k] = from_f32<T>(act_apply(to_f32<T>(v.e()[k]), act));
    stv(out + r * cols + c, o);
  }
}

template <typename T>
__global__ void __launch_bounds__(kLayThreads)
activation_kernel(T* __restrict__ out, const T* __restrict__ x, int64_t rows, int64_t cols, int64_t x_stride,
                  int act) {
  griddep_wait();
  griddep_launch_dependents();
  const int64_t n = rows * cols;
  for (int64_t i = blockIdx.x * (int64_t)kLayThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kLayThreads) {
    const int64_t r = i / cols, c = i - r * cols;
    out[i] = from_f32<T>(act_apply(to_f32<T>(x[r * x_stride + c]), act));
  }
}

// one CTA per row: pool[loc[row]] = x[row] / sqrt(mean(x[row]^2) + eps) * w   (also to `out` when given)
template <typename T>
__global__ void __launch_bounds__(kLayThreads)
rmsnorm_store_kernel(T* __restrict__ pool, T* __restrict__ out, const T* __restrict__ x, const T* __restrict__ w,
                     const int64_t* __restrict__ loc, int64_t dim, int64_t x_stride, int64_t pool_stride, float eps) {
  griddep_wait();
  griddep_launch_dependents();
  __shared__ float red[kLayThreads / 32];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * x_stride;
  float ss = 0.f;
  for (int64_t i = threadIdx.x; i < dim; i += kLayThreads) {
    const float v = to_f32<T>(xr[i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < kLayThreads / 32; ++i) tot += red[i];
  const float inv = 1.0f / sqrtf(tot / (float)dim + eps);
  T* dst = pool != nullptr ? pool + loc[row] * pool_stride : nullptr;
  for (int64_t i = threadIdx.x; i < dim; i += kLayThreads) {
    const T y = from_f32<T>(to_f32<T>(xr[i]) * inv * to_f32<T>(w[i]));
    if (dst != nullptr) dst[i] = y;
    if (out != nullptr) out[row * dim + i] = y;
  }
}

// short rows (dim <= 32 * kWarpRowMax): one warp per row, the row in registers, eight rows per CTA
constexpr int kWarpRowMax = 16;
template <typename T>
__global__ void __launch_bounds__(kLayThreads)
rmsnorm_store_warp_kernel(T* __restrict__ pool, T* __restrict__ out, const T* __restrict__ x, const T* __restrict__ w,
                          const int64_t* __restrict__ loc, int64_t rows, int64_t dim, int64_t x_stride,
                          int64_t pool_stride, float eps) {
  griddep_wait();
  griddep_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (kLayThreads / 32) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* xr = x + row * x_stride;
  float v[kWarpRowMax];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kWarpRowMax; ++j) {
    const int64_t i = (int64_t)j * 32 + lane;
    v[j] = i < dim ? to_f32<T>(xr[i]) : 0.f;
    ss += v[j] * v[j];
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
  T* dst = pool != nullptr ? pool + loc[row] * pool_stride : nullptr;
#pragma unroll
  for (int j = 0; j < kWarpRowMax; ++j) {
    const int64_t i = (int64_t)j * 32 + lane;
    if (i < dim) {
      const T y = from_f32<T>(v[j] * inv * to_f32<T>(w[i]));
      if (dst != nullptr) dst[i] = y;
      if (out != nullptr) out[row * dim + i] = y;
    }
  }
}

// out[t, h, :] = o[t, h, :] * sigmoid(g[t, h])
template <typename T>
__global__ void __launch_bounds__(kLayThreads)
head_gate_sigmoid_kernel(T* __restrict__ out, const T* __restrict__ o, const T* __restrict__ g, int64_t tokens,
                         int heads, int vdim, int64_t o_stride, int64_t g_stride) {
  griddep_wait();
  griddep_launch_dependents();
  const int64_t per_row = (int64_t)heads * vdim, n = tokens * per_row;
  for (int64_t i = blockIdx.x * (int64_t)kLayThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kLayThreads) {
    const int64_t t = i / per_row, c = i - t * per_row;
    const float gate = 1.0f / (1.0f + expf(-to_f32<T>(g[t * g_stride + c / vdim])));
    out[i] = from_f32<T>(to_f32<T>(o[t * o_stride + c]) * gate);
  }
}

// vector form: vdim and the row stride of o multiples of the vector width, 16-byte aligned pointers
template <typename T>
__global__ void __launch_bounds__(kLayThreads)
head_gate_sigmoid_vec_kernel(T* __restrict__ out, const T* __restrict__ o, const T* __restrict__ g, int64_t tokens,
                             int heads, int vdim, int64_t o_stride, int64_t g_stride) {
  griddep_wait();
  griddep_launch_dependents();
  constexpr int N = Vec16<T>::kN;
  const int64_t per_row = (int64_t)heads * vdim / N, n = tokens * per_row;
  for (int64_t i = blockIdx.x * (int64_t)kLayThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kLayThreads) {
    const int64_t t = i / per_row, c = (i - t * per_row) * N;
    const float gate = 1.0f / (1.0f + expf(-to_f32<T>(g[t * g_stride + c / vdim])));
    const Vec16<T> v = ldv(o + t * o_stride + c);
    Vec16<T> r;
#pragma unroll
    for (int k = 0; k < N; ++k) r.e()[k] = from_f32<T>(to_f32<T>(v.e()[k]) * gate);
    stv(out + t * (int64_t)heads * vdim + c, r);
  }
}

__global__ void __launch_bounds__(kLayThreads)
scale_f32_kernel(float* __restrict__ x, int64_t n, float alpha) {
  griddep_wait();
  griddep_launch_dependents();
  for (int64_t i = blockIdx.x * (int64_t)kLayThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kLayThreads)
    x[i] *= alpha;
}

inline unsigned flat_grid(int64_t n) {
  const int64_t blocks = (n + kLayThreads - 1) / kLayThreads;
  return (unsigned)(blocks < 8192 ? (blocks > 0 ? blocks : 1) : 8192);
}

}  // namespace spd

using namespace spd;

extern "C" {

int spd_embed_sincos(float* x, const void* table, const int64_t* idx, const int64_t* positions,
                     const float* freq_hi, const float* freq_lo, int64_t rows, int64_t dim, int64_t table_rows,
                     int dtype, spd_stream_t stream) {
  SPD_REQUIRE(x && table && idx && positions && freq_hi && freq_lo, SPD_E_BADARG, "spd_embed_sincos: null pointer");
  SPD_REQUIRE(rows >= 0 && dim > 0 && table_rows > 0, SPD_E_BADARG, "spd_embed_sincos: bad sizes");
  if (rows == 0) return 0;
  SPD_DISPATCH_ANY(dtype, {
    SPD_CUDA(launch(embed_sincos_kernel<T>, dim3((unsigned)rows), dim3(kLayThreads), 0, as_stream(stream),
                    pdl_enabled(), x, (const T*)table, idx, positions, freq_hi, freq_lo, dim, table_rows));
  });
  return 0;
}

int spd_cast_concat(void* out, const float* a, const float* b, int64_t rows, int64_t dim, int dtype,
                    spd_stream_t stream) {
  SPD_REQUIRE(out && a && b, SPD_E_BADARG, "spd_cast_concat: null pointer");
  SPD_REQUIRE(rows >= 0 && dim > 0, SPD_E_BADARG, "spd_cast_concat: bad sizes");
  if (rows == 0) return 0;
  SPD_DISPATCH_ANY(dtype, {
    SPD_CUDA(launch(cast_concat_kernel<T>, dim3((unsigned)rows), dim3(kLayThreads), 0, as_stream(stream),
                    pdl_enabled(), (T*)out, a, b, dim));
  });
  return 0;
}

int spd_activation(void* out, const void* x, int64_t rows, int64_t cols, int64_t x_stride, int act, int dtype,
                   spd_stream_t stream) {
  SPD_REQUIRE(out && x, SPD_E_BADARG, "spd_activation: null pointer");
  SPD_REQUIRE(rows >= 0 && cols > 0 && x_stride >= cols && act >= 0 && act <= 4, SPD_E_BADARG,
              "spd_activation: bad arguments");
  if (rows == 0) return 0;
  SPD_DISPATCH_ANY(dtype, {
    constexpr int N = 16 / (int)sizeof(T);
    if (cols % N == 0 && x_stride % N == 0 && aligned16(out) && aligned16(x)) {
      SPD_CUDA(launch(activation_vec_kernel<T>, dim3(flat_grid(rows * cols / N)), dim3(kLayThreads), 0,
                      as_stream(stream), pdl_enabled(), (T*)out, (const T*)x, rows, cols, x_stride, act));
    } else {
      SPD_CUDA(launch(activation_kernel<T>, dim3(flat_grid(rows * cols)), dim3(kLayThreads), 0, as_stream(stream),
                      pdl_enabled(), (T*)out, (const T*)x, rows, cols, x_stride, act));
    }
  });
  return 0;
}

int spd_rmsnorm_store(void* pool, void* out, const void* x, const void* w, const int64_t* loc, int64_t rows,
                      int64_t dim, int64_t x_stride, int64_t pool_stride, float eps, int dtype,
                      spd_stream_t stream) {
  SPD_REQUIRE(x && w && (pool || out) && (pool == nullptr || loc), SPD_E_BADARG, "spd_rmsnorm_store: null pointer");
  SPD_REQUIRE(rows >= 0 && dim > 0 && x_stride >= dim && (pool == nullptr || pool_stride >= dim), SPD_E_BADARG,
              "spd_rmsnorm_store: bad sizes");
  if (rows == 0) return 0;
  SPD_DISPATCH_ANY(dtype, {
    if (dim <= 32 * kWarpRowMax) {
      const int64_t ctas = (rows + kLayThreads / 32 - 1) / (kLayThreads / 32);
      SPD_CUDA(launch(rmsnorm_store_warp_kernel<T>, dim3((unsigned)ctas), dim3(kLayThreads), 0, as_stream(stream),
                      pdl_enabled(), (T*)pool, (T*)out, (const T*)x, (const T*)w, loc, rows, dim, x_stride, pool_stride,
                      eps));
    } else {
      SPD_CUDA(launch(rmsnorm_store_kernel<T>, dim3((unsigned)rows), dim3(kLayThreads), 0, as_stream(stream),
                      pdl_enabled(), (T*)pool, (T*)out, (const T*)x, (const T*)w, loc, dim, x_stride, pool_stride, eps));
    }
  });
  return 0;
}

int spd_head_gate_sigmoid(void* out, const void* o, const void* g, int64_t tokens, int heads, int vdim,
                          int64_t o_stride, int64_t g_stride, int dtype, spd_stream_t stream) {
  SPD_REQUIRE(out && o && g, SPD_E_BADARG, "spd_head_gate_sigmoid: null pointer");
  SPD_REQUIRE(tokens >= 0 && heads > 0 && vdim > 0, SPD_E_BADARG, "spd_head_gate_sigmoid: bad sizes");
  if (tokens == 0) return 0;
  SPD_DISPATCH_ANY(dtype, {
    constexpr int N = 16 / (int)sizeof(T);
    if (vdim % N == 0 && o_stride % N == 0 && aligned16(out) && aligned16(o)) {
      SPD_CUDA(launch(head_gate_sigmoid_vec_kernel<T>, dim3(flat_grid(tokens * heads * vdim / N)), dim3(kLayThreads), 0,
                      as_stream(stream), pdl_enabled(), (T*)out, (const T*)o, (const T*)g, tokens, heads, vdim,
                      o_stride, g_stride));
    } else {
      SPD_CUDA(launch(head_gate_sigmoid_kernel<T>, dim3(flat_grid(tokens * heads * vdim)), dim3(kLayThreads), 0,
                      as_stream(stream), pdl_enabled(), (T*)out, (const T*)o, (const T*)g, tokens, heads, vdim,
                      o_stride, g_stride));
    }
  });
  return 0;
}

int spd_scale_f32(float* x, int64_t n, float alpha, spd_stream_t stream) {
  SPD_REQUIRE(x, SPD_E_BADARG, "spd_scale_f32: null pointer");
  if (n <= 0) return 0;
  SPD_CUDA(launch(scale_f32_kernel, dim3(flat_grid(n)), dim3(kLayThreads), 0, as_stream(stream), pdl_enabled(), x, n,
                  alpha));
  return 0;
}

}  // extern "C"
