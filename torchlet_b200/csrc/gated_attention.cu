// What stands between the input product and the attention kernel of a mixer whose queries and keys
// are normed over the WHOLE projection and whose values may be the keys themselves.  One block per
// token; the projections arrive as float32 rows
//   proj[t] = [ q (H D) | k (G D) | ... ]
// (with separate values: [ q | k | v (G D) | ... ]).  In float32:
//   q <- q / rms(q over all H D) * wq,   k' <- k / rms(k over all G D) * wk      (plain weights);
//   the first ``dims`` entries of every head of q and k' are rotated by the token's position, entry i
//   paired with i + dims / 2: (u, v) -> (u c - v s, v c + u s), c = m cos(p f_i), s = m sin(p f_i), with
//   the frequencies f (``inv_freq``, dims / 2 floats) and the magnitude m given by the host;
//   q goes to ``q_out`` in the compute type, k' to plane 0 of the token's cache row and the value to
//   plane 1: the key AS PROJECTED (before norm and rotation) where the values are the keys.
#include <math.h>

#include "common.cuh"

namespace {

using namespace tl;

// NT threads a token: 256 up to 1,024 entries of q and k together, 512 up to 4,096, 1,024 beyond, so that a thread
// walks few entries one after the other.
template <typename T, int NT>
__global__ void __launch_bounds__(NT)
normed_qk_store_kernel(const float* __restrict__ proj, int proj_stride, const float* __restrict__ wq,
                       const float* __restrict__ wk, const float* __restrict__ inv_freq, float magnitude, float eps,
                       const int* __restrict__ positions, const int* __restrict__ token_req,
                       const int* __restrict__ block_table, int table_width, T* __restrict__ pages, int page_size,
                       int num_pages, T* __restrict__ q_out, int nh, int nkv, int d, int dims, int norm_q, int norm_k,
                       int v_offset, int write_kv) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const float* row = proj + (size_t)t * proj_stride;
  const int qn = nh * d, kn = nkv * d, half = dims >> 1;
  float ssq = 0.f, ssk = 0.f;
  for (int i = threadIdx.x; i < qn; i += NT) ssq = fmaf(row[i], row[i], ssq);
  for (int i = threadIdx.x; i < kn; i += NT) ssk = fmaf(row[qn + i], row[qn + i], ssk);
  ssq = block_sum<NT>(ssq, scratch);
  ssk = block_sum<NT>(ssk, scratch);
  const float inv_q = norm_q ? 1.f / sqrtf(ssq / (float)qn + eps) : 1.f;
  const float inv_k = norm_k ? 1.f / sqrtf(ssk / (float)kn + eps) : 1.f;
  const int pos = positions[t];
  const float p = (float)pos;

  // queries: entry e of head h; the lower entry of a rotated pair does both
  for (int c = threadIdx.x; c < qn; c += NT) {
    const int e = c % d;
    if (e >= half && e < dims) continue;
    const float a = row[c] * inv_q * (norm_q ? wq[c] : 1.f);
    if (e < half) {
      const float b = row[c + half] * inv_q * (norm_q ? wq[c + half] : 1.f);
      float sn, cs;
      sincosf(p * inv_freq[e], &sn, &cs);
      sn *= magnitude;
      cs *= magnitude;
      q_out[(size_t)t * qn + c] = from_float<T>(a * cs - b * sn);
      q_out[(size_t)t * qn + c + half] = from_float<T>(b * cs + a * sn);
    } else {
      q_out[(size_t)t * qn + c] = from_float<T>(a);
    }
  }
  if (!write_kv) return;
  int page = 0;
  if (TL_DEBUG_OK(pos / page_size < table_width, TL_DEBUG_POSITION, pos))
    page = block_table[(size_t)token_req[t] * table_width + pos / page_size];
  if (!TL_DEBUG_OK(page >= 0 && page < num_pages, TL_DEBUG_PAGE, page)) return;
  // pages: [num_pages, 2, nkv, page_size, d]
  T* kdst = pages + (size_t)page * 2 * nkv * page_size * d + (size_t)(pos % page_size) * d;
  T* vdst = kdst + (size_t)nkv * page_size * d;
  for (int c = threadIdx.x; c < kn; c += NT) {
    const int g = c / d, e = c - g * d;
    const size_t at = (size_t)g * page_size * d + e;
    vdst[at] = from_float<T>(row[v_offset + c]);
    if (e >= half && e < dims) continue;
    const float a = row[qn + c] * inv_k * (norm_k ? wk[c] : 1.f);
    if (e < half) {
      const float b = row[qn + c + half] * inv_k * (norm_k ? wk[c + half] : 1.f);
      float sn, cs;
      sincosf(p * inv_freq[e], &sn, &cs);
      sn *= magnitude;
      cs *= magnitude;
      kdst[at] = from_float<T>(a * cs - b * sn);
      kdst[at + half] = from_float<T>(b * cs + a * sn);
    } else {
      kdst[at] = from_float<T>(a);
    }
  }
}

}  // namespace

TL_DEBUG_READER(tl_gated_attention_debug_error)

extern "C" int tl_normed_qk_store(const float* proj, int proj_stride, const float* wq, const float* wk,
                                  const float* inv_freq, float magnitude, float eps, const int* positions,
                                  const int* token_req, const int* block_table, int table_width, void* pages, int dtype,
                                  int page_size, int num_pages, void* q_out, int tokens, int nh, int nkv, int d, int dims,
                                  int norm_q, int norm_k, int v_offset, int write_kv, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (d <= 0 || dims < 0 || dims > d || dims % 2 || nh <= 0 || nkv <= 0 || page_size <= 0) return TL_ERR_UNSUPPORTED;
  const long long width = (long long)(nh + nkv) * d;
#define TL_STORE(T, NT)                                                                                              \
  tl::launch_kernel(normed_qk_store_kernel<T, NT>, (unsigned)tokens, NT, 0, stream, proj, proj_stride, wq, wk, inv_freq, \
                    magnitude, eps, positions, token_req, block_table, table_width, (T*)pages, page_size, num_pages,     \
                    (T*)q_out, nh, nkv, d, dims, norm_q, norm_k, v_offset, write_kv)
  if (dtype == TL_DTYPE_F32) {
    if (width <= 1024) TL_STORE(float, 256);
    else if (width <= 4096) TL_STORE(float, 512);
    else TL_STORE(float, 1024);
  } else {
    if (width <= 1024) TL_STORE(__nv_bfloat16, 256);
    else if (width <= 4096) TL_STORE(__nv_bfloat16, 512);
    else TL_STORE(__nv_bfloat16, 1024);
  }
#undef TL_STORE
  return TL_LAUNCH_CHECK();
}
