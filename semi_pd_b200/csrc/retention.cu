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
#include "common.cuh"
#include "ptx.cuh"

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
  griddep_wait();
  griddep_launch_dependents();
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
#define SPD_RET_LAUNCH(ROWS)                                                                                     \
  SPD_CUDA(launch(retention_kernel<T, ROWS>, grid, dim3(kRetWarps * 32), smem, as_stream(stream), pdl_enabled(), o, \
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
