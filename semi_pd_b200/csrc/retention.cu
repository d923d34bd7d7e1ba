// Retention mixer: linear attention with a fixed decay per head and a matrix-valued recurrent
// state per (request, head), S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, no softmax and no
// denominator.  q and k are rotated (rotate-half pairing over the first rot_dims dimensions, fp32
// cos/sin table) and k is scaled inside the kernel, so everything that enters the recurrence is
// fp32 whatever the projections' dtype.  Decode and ragged extend (chunked prefill, mixed batches)
// are one kernel: a CTA owns (request, head, 32 value columns), keeps its [head_dim x 32] slice of
// the state in registers (rows interleaved over the warps, one column per lane), walks the
// request's new tokens in blocks of 16 staged through shared memory, and writes the state back to
// the request's slot at the end.  Every output element is summed in one fixed order (rows of a
// thread ascending, then warps ascending), so o does not depend on how a prompt was cut or batched.
// Beside attn_general.cu in role (a mixer over per-request memory); the reference has none.
// These kernels are launched WITHOUT programmatic dependent launch (plain stream order): with it,
// the prefetching form (40 KB of shared memory per CTA) between two tcgen05 GEMMs stopped making
// progress on B200 — the cause was not found, the sync form with 27 KB did not show it — and a
// mixer of a millisecond gains nothing from starting a few microseconds early.
#include "common.cuh"
#include "ptx.cuh"
#include <stdlib.h>

namespace spd {

constexpr int kRetWarps = 4;
constexpr int kRetTok = 16;   // tokens staged per block
constexpr int kRetCols = 32;  // value columns per CTA

template <typename T, int ROWS>  // ROWS = state rows per thread: head_dim <= ROWS * kRetWarps
__global__ void __launch_bounds__(kRetWarps * 32)
retention_kernel(float* __restrict__ o, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                 float* __restrict__ state, const int64_t* __restrict__ req_pool_indices,
                 const int64_t* __restrict__ seq_lens, const int64_t* __restrict__ out_cache_loc,
                 const int32_t* __restrict__ prefix_lens, const int32_t* __restrict__ extend_lens,
                 const int32_t* __restrict__ extend_start_loc, int H, int dk, int dv, int64_t q_stride,
                 int64_t k_stride, int64_t v_stride, const float* __restrict__ decay,
                 const float* __restrict__ cos_sin, int rot, int64_t max_positions, float k_scale) {
  extern __shared__ float smem[];
  float* qs = smem;                       // [kRetTok][dk]
  float* ks = qs + kRetTok * dk;          // [kRetTok][dk]
  float* vs = ks + kRetTok * dk;          // [kRetTok][kRetCols]
  float* part = vs + kRetTok * kRetCols;  // [kRetWarps][kRetTok][kRetCols]
  const int r = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.z * kRetCols + lane;
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
  const float dec = decay[h];
  float* st = state + ((int64_t)req_pool_indices[r] * H + h) * (int64_t)dk * dv;

  float S[ROWS];
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int row = warp + kRetWarps * i;
    S[i] = (pos0 > 0 && row < dk && col_ok) ? st[(int64_t)row * dv + c] : 0.f;
  }
  const int half = rot >> 1;
  for (int t0 = 0; t0 < n; t0 += kRetTok) {
    const int nt = n - t0 < kRetTok ? n - t0 : kRetTok;
    // stage rotated q, rotated + scaled k, and v of nt tokens
    for (int idx = threadIdx.x; idx < nt * dk; idx += kRetWarps * 32) {
      const int tt = idx / dk, d = idx - tt * dk;
      const int64_t row = row0 + t0 + tt;
      const T* qr = q + row * q_stride + (int64_t)h * dk;
      const T* kr = k + row * k_stride + (int64_t)h * dk;
      float qv = to_f32<T>(qr[d]), kv = to_f32<T>(kr[d]);
      if (d < rot) {
        int64_t p = pos0 + t0 + tt;
        p = p < max_positions ? p : max_positions - 1;
        const int i = d < half ? d : d - half;
        const float cs = cos_sin[p * rot + i], sn = cos_sin[p * rot + half + i];
        if (d < half) {
          qv = qv * cs - to_f32<T>(qr[d + half]) * sn;
          kv = kv * cs - to_f32<T>(kr[d + half]) * sn;
        } else {
          qv = qv * cs + to_f32<T>(qr[d - half]) * sn;
          kv = kv * cs + to_f32<T>(kr[d - half]) * sn;
        }
      }
      qs[tt * dk + d] = qv;
      ks[tt * dk + d] = kv * k_scale;
    }
    for (int idx = threadIdx.x; idx < nt * kRetCols; idx += kRetWarps * 32) {
      const int tt = idx / kRetCols, cc = idx - tt * kRetCols;
      const int col = blockIdx.z * kRetCols + cc;
      vs[idx] = col < dv ? to_f32<T>(v[(row0 + t0 + tt) * v_stride + (int64_t)h * dv + col]) : 0.f;
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float vv = vs[tt * kRetCols + lane];
      const float* kt = ks + tt * dk;
      const float* qt = qs + tt * dk;
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < ROWS; ++i) {
        const int row = warp + kRetWarps * i;
        if (row < dk) {
          S[i] = fmaf(dec, S[i], kt[row] * vv);
          acc = fmaf(S[i], qt[row], acc);
        }
      }
      part[(warp * kRetTok + tt) * kRetCols + lane] = acc;
    }
    __syncthreads();
    for (int tt = warp; tt < nt; tt += kRetWarps) {
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < kRetWarps; ++w) sum += part[(w * kRetTok + tt) * kRetCols + lane];
      if (col_ok) o[((row0 + t0 + tt) * H + h) * (int64_t)dv + c] = sum;
    }
    // the next block's staging writes qs / ks / vs (last read before the barrier above) and its
    // accumulation writes part only after the barrier that follows the staging
  }
  if (keep_state && col_ok) {
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
      const int row = warp + kRetWarps * i;
      if (row < dk) st[(int64_t)row * dv + c] = S[i];
    }
  }
}

// Prefill form of the same recurrence with the loads taken off the critical path: the raw q / k / v
// rows and the cos / sin rows of the NEXT block of 16 tokens are fetched with 16-byte cp.async into a
// raw staging area while the current block is accumulated, so a block costs its arithmetic instead
// of a chain of dependent global loads per token.  Needs 16-byte aligned rows (sizes and strides
// multiples of 16 / sizeof(T), rot_dims a multiple of 4); everything else takes retention_kernel.
// The arithmetic and its order are those of retention_kernel.
template <typename T, int ROWS>
__global__ void __launch_bounds__(kRetWarps * 32)
retention_async_kernel(float* __restrict__ o, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                       float* __restrict__ state, const int64_t* __restrict__ req_pool_indices,
                       const int32_t* __restrict__ prefix_lens, const int32_t* __restrict__ extend_lens,
                       const int32_t* __restrict__ extend_start_loc, int H, int dk, int dv, int64_t q_stride,
                       int64_t k_stride, int64_t v_stride, const float* __restrict__ decay,
                       const float* __restrict__ cos_sin, int rot, int64_t max_positions, float k_scale) {
  constexpr int N = 16 / (int)sizeof(T);
  constexpr int NT = kRetWarps * 32;
  extern __shared__ __align__(16) float smem[];
  float* qs = smem;                       // [kRetTok][dk] rotated
  float* ks = qs + kRetTok * dk;          // [kRetTok][dk] rotated, scaled
  float* vs = ks + kRetTok * dk;          // [kRetTok][kRetCols]
  float* part = vs + kRetTok * kRetCols;  // [kRetWarps][kRetTok][kRetCols]
  float* cs = part + kRetWarps * kRetTok * kRetCols;       // [kRetTok][rot] raw cos || sin rows
  T* rq = reinterpret_cast<T*>(cs + kRetTok * rot);        // [kRetTok][dk] raw
  T* rk = rq + kRetTok * dk;                               // [kRetTok][dk] raw
  T* rv = rk + kRetTok * dk;                               // [kRetTok][kRetCols] raw
  const int r = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col0 = blockIdx.z * kRetCols;
  const int c = col0 + lane;
  const bool col_ok = c < dv;
  const int64_t pos0 = prefix_lens[r];
  const int64_t row0 = extend_start_loc[r];
  const int n = extend_lens[r];
  if (n <= 0 || pos0 < 0) return;
  const float dec = decay[h];
  float* st = state + ((int64_t)req_pool_indices[r] * H + h) * (int64_t)dk * dv;
  float S[ROWS];
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int row = warp + kRetWarps * i;
    S[i] = (pos0 > 0 && row < dk && col_ok) ? st[(int64_t)row * dv + c] : 0.f;
  }
  const int half = rot >> 1;
  const int qc = dk / N, vc = kRetCols / N, cc = rot / 4;  // 16-byte chunks per row
  auto fetch = [&](int t0) {
    const int nt = n - t0 < kRetTok ? n - t0 : kRetTok;
    for (int idx = threadIdx.x; idx < nt * qc; idx += NT) {
      const int tt = idx / qc, ch = idx - tt * qc;
      const int64_t row = row0 + t0 + tt;
      cp_async16(smem_u32(rq + tt * dk + ch * N), q + row * q_stride + (int64_t)h * dk + ch * N, true);
      cp_async16(smem_u32(rk + tt * dk + ch * N), k + row * k_stride + (int64_t)h * dk + ch * N, true);
    }
    for (int idx = threadIdx.x; idx < nt * vc; idx += NT) {
      const int tt = idx / vc, ch = idx - tt * vc;
      const bool ok = col0 + ch * N < dv;  // dv is a multiple of N: a chunk is inside or outside
      cp_async16(smem_u32(rv + tt * kRetCols + ch * N),
                 v + (row0 + t0 + tt) * v_stride + (int64_t)h * dv + (ok ? col0 + ch * N : 0), ok);
    }
    for (int idx = threadIdx.x; idx < nt * cc; idx += NT) {
      const int tt = idx / cc, ch = idx - tt * cc;
      int64_t p = pos0 + t0 + tt;
      p = p < max_positions ? p : max_positions - 1;
      cp_async16(smem_u32(cs + tt * rot + ch * 4), cos_sin + p * rot + ch * 4, true);
    }
    cp_async_commit();
  };
  fetch(0);
  for (int t0 = 0; t0 < n; t0 += kRetTok) {
    const int nt = n - t0 < kRetTok ? n - t0 : kRetTok;
    cp_async_wait<0>();
    __syncthreads();  // raw rows of this block visible; the previous block's reduce has finished
    for (int idx = threadIdx.x; idx < nt * dk; idx += NT) {
      const int tt = idx / dk, d = idx - tt * dk;
      float qv = to_f32<T>(rq[idx]), kv = to_f32<T>(rk[idx]);
      if (d < rot) {
        const int i = d < half ? d : d - half;
        const float cv = cs[tt * rot + i], sn = cs[tt * rot + half + i];
        if (d < half) {
          qv = qv * cv - to_f32<T>(rq[idx + half]) * sn;
          kv = kv * cv - to_f32<T>(rk[idx + half]) * sn;
        } else {
          qv = qv * cv + to_f32<T>(rq[idx - half]) * sn;
          kv = kv * cv + to_f32<T>(rk[idx - half]) * sn;
        }
      }
      qs[idx] = qv;
      ks[idx] = kv * k_scale;
    }
    for (int idx = threadIdx.x; idx < nt * kRetCols; idx += NT) vs[idx] = to_f32<T>(rv[idx]);
    __syncthreads();  // staging complete; the raw area is free again
    if (t0 + kRetTok < n) fetch(t0 + kRetTok);
    for (int tt = 0; tt < nt; ++tt) {
      const float vv = vs[tt * kRetCols + lane];
      const float* kt = ks + tt * dk;
      const float* qt = qs + tt * dk;
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < ROWS; ++i) {
        const int row = warp + kRetWarps * i;
        if (row < dk) {
          S[i] = fmaf(dec, S[i], kt[row] * vv);
          acc = fmaf(S[i], qt[row], acc);
        }
      }
      part[(warp * kRetTok + tt) * kRetCols + lane] = acc;
    }
    __syncthreads();
    for (int tt = warp; tt < nt; tt += kRetWarps) {
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < kRetWarps; ++w) sum += part[(w * kRetTok + tt) * kRetCols + lane];
      if (col_ok) o[((row0 + t0 + tt) * H + h) * (int64_t)dv + c] = sum;
    }
  }
  if (col_ok) {
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
      const int row = warp + kRetWarps * i;
      if (row < dk) st[(int64_t)row * dv + c] = S[i];
    }
  }
}

}  // namespace spd

using namespace spd;

extern "C" {

int spd_retention(float* o, const void* q, const void* k, const void* v, float* state,
                  const int64_t* req_pool_indices, const int64_t* seq_lens, const int64_t* out_cache_loc,
                  const int32_t* prefix_lens, const int32_t* extend_lens, const int32_t* extend_start_loc,
                  int64_t batch, int num_heads, int head_dim, int v_dim, int64_t q_stride, int64_t k_stride,
                  int64_t v_stride, const float* decay, const float* cos_sin, int rot_dims,
                  int64_t max_positions, float k_scale, int dtype, spd_stream_t stream) {
  SPD_REQUIRE(o && q && k && v && state && req_pool_indices && decay, SPD_E_BADARG, "spd_retention: null pointer");
  SPD_REQUIRE(seq_lens != nullptr || (prefix_lens && extend_lens && extend_start_loc), SPD_E_BADARG,
              "spd_retention: extend needs prefix_lens, extend_lens and extend_start_loc");
  SPD_REQUIRE(num_heads > 0 && head_dim > 0 && head_dim <= 64 * kRetWarps && v_dim > 0, SPD_E_SHAPE,
              "spd_retention: head_dim %d above %d", head_dim, 64 * kRetWarps);
  SPD_REQUIRE(rot_dims >= 0 && rot_dims <= head_dim && rot_dims % 2 == 0 && (rot_dims == 0 || (cos_sin && max_positions > 0)),
              SPD_E_BADARG, "spd_retention: bad rotation (rot_dims %d)", rot_dims);
  if (batch == 0) return 0;
  const dim3 grid((unsigned)batch, (unsigned)num_heads, (unsigned)((v_dim + kRetCols - 1) / kRetCols));
  const size_t smem = sizeof(float) * ((size_t)2 * kRetTok * head_dim + kRetTok * kRetCols + kRetWarps * kRetTok * kRetCols);
  // ragged extend with 16-byte aligned rows: the prefetching form
  const int vecn = dtype == SPD_F32 ? 4 : 8;
  const bool async_ok = seq_lens == nullptr && head_dim % vecn == 0 && v_dim % vecn == 0 && q_stride % vecn == 0 &&
                        k_stride % vecn == 0 && v_stride % vecn == 0 && rot_dims % 4 == 0 && aligned16(q) &&
                        aligned16(k) && aligned16(v) && (rot_dims == 0 || aligned16(cos_sin)) &&
                        getenv("SPD_RETENTION_SYNC") == nullptr;
  const size_t esz = dtype == SPD_F32 ? 4 : 2;
  const size_t smem_async = smem + sizeof(float) * kRetTok * (size_t)rot_dims + esz * kRetTok * (2 * (size_t)head_dim + kRetCols);
#define SPD_RET_LAUNCH_ASYNC(ROWS)                                                                                  \
  do {                                                                                                              \
    static size_t configured = 0;                                                                                   \
    if (smem_async > 48 * 1024 && smem_async > configured) {                                                        \
      SPD_CUDA(cudaFuncSetAttribute(retention_async_kernel<T, ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                    (int)smem_async));                                                              \
      configured = smem_async;                                                                                      \
    }                                                                                                               \
    SPD_CUDA(launch(retention_async_kernel<T, ROWS>, grid, dim3(kRetWarps * 32), smem_async, as_stream(stream),     \
                    /*pdl=*/false, o, (const T*)q, (const T*)k, (const T*)v, state, req_pool_indices, prefix_lens,  \
                    extend_lens, extend_start_loc, num_heads, head_dim, v_dim, q_stride, k_stride, v_stride, decay, \
                    cos_sin, rot_dims, max_positions, k_scale));                                                    \
  } while (0)
  if (async_ok) {
    SPD_DISPATCH_ANY(dtype, {
      if (head_dim <= 8 * kRetWarps) SPD_RET_LAUNCH_ASYNC(8);
      else if (head_dim <= 16 * kRetWarps) SPD_RET_LAUNCH_ASYNC(16);
      else if (head_dim <= 32 * kRetWarps) SPD_RET_LAUNCH_ASYNC(32);
      else SPD_RET_LAUNCH_ASYNC(64);
    });
    return 0;
  }
#undef SPD_RET_LAUNCH_ASYNC
#define SPD_RET_LAUNCH(ROWS)                                                                                     \
  SPD_CUDA(launch(retention_kernel<T, ROWS>, grid, dim3(kRetWarps * 32), smem, as_stream(stream), /*pdl=*/false, o, \
                  (const T*)q, (const T*)k, (const T*)v, state, req_pool_indices, seq_lens, out_cache_loc,       \
                  prefix_lens, extend_lens, extend_start_loc, num_heads, head_dim, v_dim, q_stride, k_stride,    \
                  v_stride, decay, cos_sin, rot_dims, max_positions, k_scale))
  SPD_DISPATCH_ANY(dtype, {
    if (head_dim <= 8 * kRetWarps) SPD_RET_LAUNCH(8);
    else if (head_dim <= 16 * kRetWarps) SPD_RET_LAUNCH(16);
    else if (head_dim <= 32 * kRetWarps) SPD_RET_LAUNCH(32);
    else SPD_RET_LAUNCH(64);
  });
#undef SPD_RET_LAUNCH
  return 0;
}

}  // extern "C"
