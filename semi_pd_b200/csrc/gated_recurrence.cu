// Linear attention with a data-dependent decay per key channel, and the token shift that feeds
// one form of it.  Per (request, head) a matrix state S [head_dim x v_dim] in fp32 is carried from
// token to token:
//
//   form 0 (gated linear attention)   w_t = sigmoid(z_t)^(1/tau)
//                                     S_t = diag(w_t) S_(t-1) + k_t v_t^T ;  o_t = S_t^T (q_t * q_scale)
//   form 1 (time mixing with a bonus) w_t = exp(-exp(z_t))
//                                     o_t = (S_(t-1) + diag(u) k_t v_t^T)^T q_t ;  S_t = diag(w_t) S_(t-1) + k_t v_t^T
//
// z is the raw output of the decay projection (any dtype) plus an fp32 bias; the decay itself, the
// products and the state are fp32 in every dtype.  Decode and ragged extend (chunked prefill, mixed
// batches) are one kernel with the layout of retention.cu: a CTA owns (request, head, 32 value
// columns), warp w holds state rows w * ROWS .. and lane l the column l; the request's new tokens
// are walked in blocks staged through shared memory (q, k and the decay of a block, rows zero-padded),
// the warps' partial outputs meet in shared memory once per block, and every output element is
// summed in one fixed order (rows of a thread ascending over two interleaved accumulators, then
// warps ascending), so o does not depend on how a prompt was cut or batched.  A request that starts
// at position 0 ignores what its state slot held before.  Plain stream order (no programmatic
// dependent launch), as retention.cu.
//
// token_shift_mix: out_s[t] = h[t] + (h[t-1] - h[t]) * mu_s for several s at once, h[-1] of a request
// being the row its state slot keeps (zeros at position 0); the slot then receives the request's last
// row.  The CTA that reads a slot is the one that writes it, so one launch does both.
#include "common.cuh"
#include "ptx.cuh"
#include <stdlib.h>

namespace spd {

constexpr int kGrTok = 16;   // tokens staged per block (extend); decode stages its one token
constexpr int kGrCols = 32;  // value columns per CTA

__device__ __forceinline__ float decay_sigmoid_pow(float z, float inv_tau) {
  // sigmoid(z)^(1/tau) = exp(-softplus(-z) / tau), softplus evaluated without overflow
  const float sp = z < 0.f ? -z + log1pf(expf(z)) : log1pf(expf(-z));
  return expf(-sp * inv_tau);
}
__device__ __forceinline__ float decay_double_exp(float z) { return expf(-expf(z)); }

template <typename T, int W, int ROWS, int TOK, int FORM, bool ASYNC>
__global__ void __launch_bounds__(W * 32)
gated_recurrence_kernel(float* __restrict__ o, const T* __restrict__ q, const T* __restrict__ k,
                        const T* __restrict__ v, const T* __restrict__ z, float* __restrict__ state,
                        const int64_t* __restrict__ req_pool_indices, const int64_t* __restrict__ seq_lens,
                        const int64_t* __restrict__ out_cache_loc, const int32_t* __restrict__ prefix_lens,
                        const int32_t* __restrict__ extend_lens, const int32_t* __restrict__ extend_start_loc, int H,
                        int dk, int dv, int64_t q_stride, int64_t k_stride, int64_t v_stride, int64_t z_stride,
                        const float* __restrict__ z_bias, const float* __restrict__ bonus, float q_scale,
                        float inv_tau) {
  static_assert(ROWS % 4 == 0, "rows per thread are read as float4");
  constexpr int DKP = W * ROWS;  // padded head_dim
  constexpr int NT = W * 32;
  extern __shared__ __align__(16) float smem[];
  float* qs = smem;                    // [TOK][DKP] scaled
  float* ks = qs + TOK * DKP;          // [TOK][DKP]
  float* ws = ks + TOK * DKP;          // [TOK][DKP] decay
  float* vs = ws + TOK * DKP;          // [TOK][kGrCols]
  float* part = vs + TOK * kGrCols;    // [W][TOK][kGrCols]
  T* rq = reinterpret_cast<T*>(part + W * TOK * kGrCols);  // ASYNC: [TOK][dk] raw rows of the NEXT block
  T* rk = rq + TOK * dk;                                   // ASYNC: [TOK][dk]
  T* rz = rk + TOK * dk;                                   // ASYNC: [TOK][dk]
  T* rv = rz + TOK * dk;                                   // ASYNC: [TOK][kGrCols]
  constexpr int N = 16 / (int)sizeof(T);
  const int r = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col0 = blockIdx.z * kGrCols;
  const int c = col0 + lane;
  const bool col_ok = c < dv;

  int64_t pos0, row0;
  int n;
  bool keep_state = true;
  if (seq_lens != nullptr) {
    pos0 = seq_lens[r] - 1;
    row0 = r;
    n = 1;
    if (out_cache_loc != nullptr && out_cache_loc[r] == 0) keep_state = false;  // padded row of a captured batch
  } else {
    pos0 = prefix_lens[r];
    row0 = extend_start_loc[r];
    n = extend_lens[r];
  }
  if (n <= 0 || pos0 < 0) return;
  float* st = state + ((int64_t)req_pool_indices[r] * H + h) * (int64_t)dk * dv;

  float S[ROWS], U[ROWS];
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int row = warp * ROWS + i;
    S[i] = (pos0 > 0 && row < dk && col_ok) ? st[(int64_t)row * dv + c] : 0.f;
    U[i] = (FORM == 1 && row < dk) ? bonus[h * dk + row] : 0.f;
  }
  // ASYNC (ragged extend with 16-byte aligned rows): the raw q / k / z / v rows of the next block arrive by
  // 16-byte cp.async while the current block is accumulated
  const int qc = dk / N, vc = kGrCols / N;
  auto fetch = [&](int t0) {
    const int nt = n - t0 < TOK ? n - t0 : TOK;
    for (int idx = threadIdx.x; idx < nt * qc; idx += NT) {
      const int tt = idx / qc, ch = idx - tt * qc;
      const int64_t row = row0 + t0 + tt;
      cp_async16(smem_u32(rq + tt * dk + ch * N), q + row * q_stride + (int64_t)h * dk + ch * N, true);
      cp_async16(smem_u32(rk + tt * dk + ch * N), k + row * k_stride + (int64_t)h * dk + ch * N, true);
      cp_async16(smem_u32(rz + tt * dk + ch * N), z + row * z_stride + (int64_t)h * dk + ch * N, true);
    }
    for (int idx = threadIdx.x; idx < nt * vc; idx += NT) {
      const int tt = idx / vc, ch = idx - tt * vc;
      const bool ok = col0 + ch * N < dv;  // dv is a multiple of N: a chunk is inside or outside
      cp_async16(smem_u32(rv + tt * kGrCols + ch * N),
                 v + (row0 + t0 + tt) * v_stride + (int64_t)h * dv + (ok ? col0 + ch * N : 0), ok);
    }
    cp_async_commit();
  };
  if (ASYNC) fetch(0);
  for (int t0 = 0; t0 < n; t0 += TOK) {
    const int nt = n - t0 < TOK ? n - t0 : TOK;
    if (ASYNC) {
      cp_async_wait<0>();
      __syncthreads();  // raw rows of this block visible; the previous block's reduce has finished
    }
    for (int idx = threadIdx.x; idx < nt * DKP; idx += NT) {
      const int tt = idx / DKP, d = idx - tt * DKP;
      float qv = 0.f, kv = 0.f, wv = 0.f;
      if (d < dk) {
        const int64_t row = row0 + t0 + tt;
        float zz;
        if (ASYNC) {
          qv = to_f32<T>(rq[tt * dk + d]) * q_scale;
          kv = to_f32<T>(rk[tt * dk + d]);
          zz = to_f32<T>(rz[tt * dk + d]);
        } else {
          qv = to_f32<T>(q[row * q_stride + (int64_t)h * dk + d]) * q_scale;
          kv = to_f32<T>(k[row * k_stride + (int64_t)h * dk + d]);
          zz = to_f32<T>(z[row * z_stride + (int64_t)h * dk + d]);
        }
        if (z_bias != nullptr) zz += z_bias[h * dk + d];
        wv = FORM == 0 ? decay_sigmoid_pow(zz, inv_tau) : decay_double_exp(zz);
      }
      qs[idx] = qv;
      ks[idx] = kv;
      ws[idx] = wv;
    }
    for (int idx = threadIdx.x; idx < nt * kGrCols; idx += NT) {
      const int tt = idx / kGrCols, cl = idx - tt * kGrCols;
      if (ASYNC) vs[idx] = to_f32<T>(rv[idx]);  // chunks outside the row were zero-filled
      else vs[idx] = col0 + cl < dv ? to_f32<T>(v[(row0 + t0 + tt) * v_stride + (int64_t)h * dv + col0 + cl]) : 0.f;
    }
    __syncthreads();  // staging complete (ASYNC: the raw area is free again)
    if (ASYNC && t0 + TOK < n) fetch(t0 + TOK);
    for (int tt = 0; tt < nt; ++tt) {
      const float vv = vs[tt * kGrCols + lane];
      const float4* kt = reinterpret_cast<const float4*>(ks + tt * DKP + warp * ROWS);
      const float4* qt = reinterpret_cast<const float4*>(qs + tt * DKP + warp * ROWS);
      const float4* wt = reinterpret_cast<const float4*>(ws + tt * DKP + warp * ROWS);
      float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
      for (int i = 0; i < ROWS / 4; ++i) {
        const float4 k4 = kt[i], q4 = qt[i], w4 = wt[i];
        const float kk[4] = {k4.x, k4.y, k4.z, k4.w};
        const float qq[4] = {q4.x, q4.y, q4.z, q4.w};
        const float ww[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float kv = kk[j] * vv;
          float& acc = (j & 1) ? acc1 : acc0;
          if (FORM == 0) {
            S[4 * i + j] = fmaf(ww[j], S[4 * i + j], kv);
            acc = fmaf(S[4 * i + j], qq[j], acc);
          } else {
            acc = fmaf(fmaf(U[4 * i + j], kv, S[4 * i + j]), qq[j], acc);
            S[4 * i + j] = fmaf(ww[j], S[4 * i + j], kv);
          }
        }
      }
      part[(warp * TOK + tt) * kGrCols + lane] = acc0 + acc1;
    }
    __syncthreads();
    for (int tt = warp; tt < nt; tt += W) {
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < W; ++w) sum += part[(w * TOK + tt) * kGrCols + lane];
      if (col_ok) o[((row0 + t0 + tt) * H + h) * (int64_t)dv + c] = sum;
    }
    // the next block's staging writes qs / ks / ws / vs, last read before the barrier above; its
    // accumulation writes part only after the barrier that follows the staging
  }
  if (keep_state && col_ok) {
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
      const int row = warp * ROWS + i;
      if (row < dk) st[(int64_t)row * dv + c] = S[i];
    }
  }
}

template <typename T, int W, int ROWS, int TOK, int FORM, bool ASYNC>
int gated_recurrence_launch(dim3 grid, cudaStream_t stream, float* o, const void* q, const void* k, const void* v,
                            const void* z, float* state, const int64_t* req_pool_indices, const int64_t* seq_lens,
                            const int64_t* out_cache_loc, const int32_t* prefix_lens, const int32_t* extend_lens,
                            const int32_t* extend_start_loc, int H, int dk, int dv, int64_t q_stride, int64_t k_stride,
                            int64_t v_stride, int64_t z_stride, const float* z_bias, const float* bonus, float q_scale,
                            float inv_tau) {
  const size_t smem = sizeof(float) * ((size_t)3 * TOK * W * ROWS + TOK * kGrCols + (size_t)W * TOK * kGrCols) +
                      (ASYNC ? sizeof(T) * TOK * (3 * (size_t)dk + kGrCols) : 0);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    SPD_CUDA(cudaFuncSetAttribute(gated_recurrence_kernel<T, W, ROWS, TOK, FORM, ASYNC>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  SPD_CUDA(launch(gated_recurrence_kernel<T, W, ROWS, TOK, FORM, ASYNC>, grid, dim3(W * 32), smem, stream, /*pdl=*/false, o,
                  (const T*)q, (const T*)k, (const T*)v, (const T*)z, state, req_pool_indices, seq_lens, out_cache_loc,
                  prefix_lens, extend_lens, extend_start_loc, H, dk, dv, q_stride, k_stride, v_stride, z_stride, z_bias,
                  bonus, q_scale, inv_tau));
  return 0;
}

// ------------------------------------------------------------------------------------------------
// token shift: one CTA per (request, slice of the row, chunk of the request's new rows)
// ------------------------------------------------------------------------------------------------
constexpr int kShiftThreads = 128;
constexpr int kShiftMaxMix = 8;  // mixes per launch
constexpr int kShiftChunk = 32;  // rows a CTA walks

// VEC elements per thread: 16-byte vectors where the row size and the pointers allow, else one element
template <typename T, int VEC>
__global__ void __launch_bounds__(kShiftThreads)
token_shift_mix_kernel(T* __restrict__ out, const T* __restrict__ h, const T* __restrict__ mu,
                       float* __restrict__ shift_state, const int64_t* __restrict__ req_pool_indices,
                       const int64_t* __restrict__ seq_lens, const int64_t* __restrict__ out_cache_loc,
                       const int32_t* __restrict__ prefix_lens, const int32_t* __restrict__ extend_lens,
                       const int32_t* __restrict__ extend_start_loc, int64_t total_rows, int64_t dim, int n_mix) {
  const int r = blockIdx.x;
  const int64_t i = ((int64_t)blockIdx.y * kShiftThreads + threadIdx.x) * VEC;
  if (i >= dim) return;
  int64_t pos0, row0;
  int n;
  bool keep_state = true;
  if (seq_lens != nullptr) {
    pos0 = seq_lens[r] - 1;
    row0 = r;
    n = 1;
    if (out_cache_loc != nullptr && out_cache_loc[r] == 0) keep_state = false;
  } else {
    pos0 = prefix_lens[r];
    row0 = extend_start_loc[r];
    n = extend_lens[r];
  }
  const int t_lo = blockIdx.z * kShiftChunk;
  if (n <= 0 || pos0 < 0 || t_lo >= n) return;
  const int t_hi = t_lo + kShiftChunk < n ? t_lo + kShiftChunk : n;
  auto load = [&](const T* p, float* dst) {
    if constexpr (VEC == 1) {
      dst[0] = to_f32<T>(p[0]);
    } else {
      const Vec16<T> v = ldv(p);
#pragma unroll
      for (int e = 0; e < VEC; ++e) dst[e] = to_f32<T>(v.e()[e]);
    }
  };
  float prev[VEC], cur[VEC];
  if (t_lo == 0) {
    // the request's first new row: its predecessor is what the slot keeps (nothing at position 0).  This
    // thread is the only reader of these slot elements in the launch, and writes them right after: the
    // request's last row.
    float* slot = shift_state + (int64_t)req_pool_indices[r] * dim + i;
#pragma unroll
    for (int e = 0; e < VEC; ++e) prev[e] = pos0 > 0 ? slot[e] : 0.f;
    if (keep_state) {
      load(h + (row0 + n - 1) * dim + i, cur);
#pragma unroll
      for (int e = 0; e < VEC; ++e) slot[e] = cur[e];
    }
  } else {
    load(h + (row0 + t_lo - 1) * dim + i, prev);
  }
  for (int t = t_lo; t < t_hi; ++t) {
    load(h + (row0 + t) * dim + i, cur);
    for (int s = 0; s < n_mix; ++s) {
      float m[VEC];
      load(mu + (int64_t)s * dim + i, m);
      T* dst = out + ((int64_t)s * total_rows + row0 + t) * dim + i;
      if constexpr (VEC == 1) {
        dst[0] = from_f32<T>(fmaf(prev[0] - cur[0], m[0], cur[0]));
      } else {
        Vec16<T> o;
#pragma unroll
        for (int e = 0; e < VEC; ++e) o.e()[e] = from_f32<T>(fmaf(prev[e] - cur[e], m[e], cur[e]));
        stv(dst, o);
      }
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) prev[e] = cur[e];
  }
}

}  // namespace spd

using namespace spd;

extern "C" {

int spd_gated_recurrence(float* o, const void* q, const void* k, const void* v, const void* z, float* state,
                         const int64_t* req_pool_indices, const int64_t* seq_lens, const int64_t* out_cache_loc,
                         const int32_t* prefix_lens, const int32_t* extend_lens, const int32_t* extend_start_loc,
                         int64_t batch, int num_heads, int head_dim, int v_dim, int64_t q_stride, int64_t k_stride,
                         int64_t v_stride, int64_t z_stride, const float* z_bias, const float* bonus, int form,
                         float q_scale, float tau, int dtype, spd_stream_t stream) {
  SPD_REQUIRE(o && q && k && v && z && state && req_pool_indices, SPD_E_BADARG, "spd_gated_recurrence: null pointer");
  SPD_REQUIRE(seq_lens != nullptr || (prefix_lens && extend_lens && extend_start_loc), SPD_E_BADARG,
              "spd_gated_recurrence: extend needs prefix_lens, extend_lens and extend_start_loc");
  SPD_REQUIRE(num_heads > 0 && num_heads <= 65535 && head_dim > 0 && head_dim <= 256 && v_dim > 0, SPD_E_SHAPE,
              "spd_gated_recurrence: head_dim %d above 256", head_dim);
  SPD_REQUIRE(form == 0 || (form == 1 && bonus != nullptr), SPD_E_BADARG, "spd_gated_recurrence: form %d", form);
  SPD_REQUIRE(form == 1 || tau > 0.f, SPD_E_BADARG, "spd_gated_recurrence: tau must be positive");
  if (batch == 0) return 0;
  const dim3 grid((unsigned)batch, (unsigned)num_heads, (unsigned)((v_dim + kGrCols - 1) / kGrCols));
  const bool decode = seq_lens != nullptr;
  const float inv_tau = form == 0 ? 1.0f / tau : 0.f;
  // ragged extend with 16-byte aligned rows: the prefetching form
  const int vecn = dtype == SPD_F32 ? 4 : 8;
  const bool async_ok = !decode && head_dim % vecn == 0 && v_dim % vecn == 0 && q_stride % vecn == 0 &&
                        k_stride % vecn == 0 && v_stride % vecn == 0 && z_stride % vecn == 0 && aligned16(q) &&
                        aligned16(k) && aligned16(v) && aligned16(z) && getenv("SPD_RECURRENCE_SYNC") == nullptr;
#define SPD_GR_ARGS                                                                                               \
  grid, as_stream(stream), o, q, k, v, z, state, req_pool_indices, seq_lens, out_cache_loc, prefix_lens,          \
      extend_lens, extend_start_loc, num_heads, head_dim, v_dim, q_stride, k_stride, v_stride, z_stride, z_bias,  \
      bonus, q_scale, inv_tau
#define SPD_GR_FORM(W, ROWS, TOK, ASYNC)                                                     \
  return form == 0 ? gated_recurrence_launch<T, W, ROWS, TOK, 0, ASYNC>(SPD_GR_ARGS)          \
                   : gated_recurrence_launch<T, W, ROWS, TOK, 1, ASYNC>(SPD_GR_ARGS)
#define SPD_GR_SHAPE(W, ROWS)                            \
  do {                                                   \
    if (decode) SPD_GR_FORM(W, ROWS, 1, false);          \
    else if (async_ok) SPD_GR_FORM(W, ROWS, kGrTok, true); \
    else SPD_GR_FORM(W, ROWS, kGrTok, false);            \
  } while (0)
  SPD_DISPATCH_ANY(dtype, {
    if (head_dim <= 32) SPD_GR_SHAPE(4, 8);
    else if (head_dim <= 64) SPD_GR_SHAPE(8, 8);
    else if (head_dim <= 128) SPD_GR_SHAPE(16, 8);
    else SPD_GR_SHAPE(16, 16);
  });
#undef SPD_GR_SHAPE
#undef SPD_GR_FORM
#undef SPD_GR_ARGS
  return 0;
}

int spd_token_shift_mix(void* out, const void* h, const void* mu, float* shift_state,
                        const int64_t* req_pool_indices, const int64_t* seq_lens, const int64_t* out_cache_loc,
                        const int32_t* prefix_lens, const int32_t* extend_lens, const int32_t* extend_start_loc,
                        int64_t batch, int64_t total_rows, int64_t max_rows_per_request, int64_t dim, int n_mix,
                        int dtype, spd_stream_t stream) {
  SPD_REQUIRE(out && h && mu && shift_state && req_pool_indices, SPD_E_BADARG, "spd_token_shift_mix: null pointer");
  SPD_REQUIRE(seq_lens != nullptr || (prefix_lens && extend_lens && extend_start_loc), SPD_E_BADARG,
              "spd_token_shift_mix: extend needs prefix_lens, extend_lens and extend_start_loc");
  SPD_REQUIRE(dim > 0 && n_mix > 0 && n_mix <= kShiftMaxMix, SPD_E_SHAPE, "spd_token_shift_mix: %d mixes (max %d)",
              n_mix, kShiftMaxMix);
  if (batch == 0 || total_rows == 0) return 0;
  // max_rows_per_request: a host-side bound of extend_lens (decode: 1)
  const int64_t rows = seq_lens != nullptr ? 1 : (max_rows_per_request > 0 ? max_rows_per_request : total_rows);
  const int64_t chunks = (rows + kShiftChunk - 1) / kShiftChunk;
  SPD_REQUIRE(chunks <= 65535 && (dim + kShiftThreads - 1) / kShiftThreads <= 65535, SPD_E_SHAPE,
              "spd_token_shift_mix: too many rows per request");
  SPD_DISPATCH_ANY(dtype, {
    constexpr int N = 16 / (int)sizeof(T);
    if (dim % N == 0 && aligned16(out) && aligned16(h) && aligned16(mu)) {
      const int64_t per = (int64_t)kShiftThreads * N;
      const dim3 grid((unsigned)batch, (unsigned)((dim + per - 1) / per), (unsigned)chunks);
      SPD_CUDA(launch(token_shift_mix_kernel<T, N>, grid, dim3(kShiftThreads), 0, as_stream(stream), /*pdl=*/false,
                      (T*)out, (const T*)h, (const T*)mu, shift_state, req_pool_indices, seq_lens, out_cache_loc,
                      prefix_lens, extend_lens, extend_start_loc, total_rows, dim, n_mix));
    } else {
      const dim3 grid((unsigned)batch, (unsigned)((dim + kShiftThreads - 1) / kShiftThreads), (unsigned)chunks);
      SPD_CUDA(launch(token_shift_mix_kernel<T, 1>, grid, dim3(kShiftThreads), 0, as_stream(stream), /*pdl=*/false,
                      (T*)out, (const T*)h, (const T*)mu, shift_state, req_pool_indices, seq_lens, out_cache_loc,
                      prefix_lens, extend_lens, extend_start_loc, total_rows, dim, n_mix));
    }
  });
  return 0;
}

}  // extern "C"
