// Latent-space attention on the tensor cores (bfloat16, mma.sync.m16n8k16, float32 accumulators).
//
// All heads of a token read the same cached rows [c (dv) | k_rot] (dk = dv + rot entries), so the
// (token, head) pairs of a request are packed into row tiles of 64 and a CTA multiplies one row
// tile with the request's cached rows, 64 keys at a time:
//
//   S = Q K^T   (64 x dk by dk x 64),  online softmax in float32,  O += P V  with V = K[:, :dv].
//
// A CTA has 4 x NCW warps: warp (rw, cw) owns rows 16 rw .. 16 rw + 15.  For S it takes the key
// columns [cw 64/NCW, (cw + 1) 64/NCW) of the tile, so that S is computed once; row maxima and sums
// of the NCW warps of a row block meet in shared memory, P goes to shared memory in bfloat16, and
// for O every warp reads all of P and the value columns [cw DVW, (cw + 1) DVW) that it accumulates
// (DVW <= 128: 64 float registers a thread).  NCW = 1, 2, 4 for dv up to 128, 256, 512.
// Rows of keys past the tile's last visible key are zero-filled (0 x stale NaN would be NaN).
//
// Requests that bring one token (decode) may split their keys over gridDim.y CTAs; every split
// leaves an unnormalized partial result (O, max, sum) and a second kernel merges them.  How many
// key tiles a split takes follows from the request's own length on the device, so a captured
// step planned for the engine's length limit is valid for every length.
//
// Q: [T, heads, dk] bfloat16 (absorbed queries);  cache layer: [page][slot in page][dk];
// out: [T, heads, dv] bfloat16.
#include <math.h>

#include "common.cuh"

namespace {

using namespace tl;

constexpr int ROWS = 64, KEYS = 64, PAD = 8, P_STRIDE = KEYS + PAD;

__device__ __forceinline__ void copy16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void copies_done() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void load_frag(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void load_frag_t(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct Args {
  const __nv_bfloat16* q;
  const __nv_bfloat16* pages;
  const int* block_table;
  const int* req_indptr;
  const int* kv_before;
  const int* tile_req;   // null: every request brings one token; tile i belongs to request i / tiles_per_req
  const int* tile_row;   // first packed row of the tile inside its request
  __nv_bfloat16* out;
  float* part_o;         // [T heads][splits][dv]   (splits > 1)
  float* part_ml;        // [T heads][splits][2]
  int table_width, heads, dk, dv, page_size, num_pages, tiles_per_req, splits;
  float scale;
};

template <int NCW>
__global__ void __launch_bounds__(128 * NCW)
latent_attention_mma_kernel(const Args a) {
  tl::pdl_wait();
  tl::pdl_launch_dependents();
  constexpr int KW = KEYS / NCW;  // key columns of S a warp computes
  constexpr int SNT = KW / 8;     // its n-tiles of S
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int stride = a.dk + PAD;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* Ks = Qs + (size_t)ROWS * stride;
  __nv_bfloat16* Ps = Ks + (size_t)KEYS * stride;
  float* red_max = reinterpret_cast<float*>(Ps + ROWS * P_STRIDE);  // [NCW][ROWS]
  float* red_sum = red_max + NCW * ROWS;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rw = warp & 3, cw = warp >> 2;
  const int g = lane >> 2, t4 = lane & 3;
  const int tile = blockIdx.x, split = blockIdx.y;
  const int req = a.tile_req ? a.tile_req[tile] : tile / a.tiles_per_req;
  const int row0 = a.tile_req ? a.tile_row[tile] : (tile % a.tiles_per_req) * ROWS;
  const int first_token = a.req_indptr[req];
  const int rows_total = (a.req_indptr[req + 1] - first_token) * a.heads;
  const int nrows = rows_total - row0 < ROWS ? rows_total - row0 : ROWS;
  const int kvb = a.kv_before[req];
  const int kv_end = kvb + (row0 + nrows - 1) / a.heads + 1;  // keys the tile's last row sees
  const int key_tiles = (kv_end + KEYS - 1) / KEYS;
  int tile_lo = 0, tile_hi = key_tiles;
  if (a.splits > 1) {
    const int per = (key_tiles + a.splits - 1) / a.splits;
    tile_lo = split * per;
    tile_hi = tile_lo + per < key_tiles ? tile_lo + per : key_tiles;
  }
  const int* table = a.block_table + (size_t)req * a.table_width;
  const size_t q_row0 = (size_t)first_token * a.heads + row0;  // global packed row of the tile's first row

  // the query rows
  const int chunks = a.dk >> 3;
  for (int e = tid; e < ROWS * chunks; e += 128 * NCW) {
    const int r = e / chunks, c = e - r * chunks;
    copy16(Qs + (size_t)r * stride + c * 8, a.q + (q_row0 + (r < nrows ? r : 0)) * a.dk + c * 8, r < nrows);
  }

  // value columns of this warp: n-tiles [nt_lo, nt_hi) of 8 columns
  const int dv_tiles = a.dv >> 3;
  int per_warp = ((dv_tiles + NCW - 1) / NCW + 1) & ~1;  // an even number of n-tiles (loaded in pairs)
  const int nt_lo = cw * per_warp;
  const int nt_cnt = nt_lo >= dv_tiles ? 0 : (dv_tiles - nt_lo < per_warp ? dv_tiles - nt_lo : per_warp);

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int r_lo = rw * 16 + g, r_hi = r_lo + 8;
  const int pos_lo = kvb + (row0 + r_lo) / a.heads, pos_hi = kvb + (row0 + r_hi) / a.heads;
  const bool on_lo = r_lo < nrows, on_hi = r_hi < nrows;
  const bool warp_has_rows = rw * 16 < nrows;  // a tile of few rows (single tokens, few heads): the other warps only load

  for (int kt = tile_lo; kt < tile_hi; ++kt) {
    const int key0 = kt * KEYS;
    __syncthreads();  // everyone is done with Ks and Ps of the tile before
    for (int e = tid; e < KEYS * chunks; e += 128 * NCW) {
      const int r = e / chunks, c = e - r * chunks;
      const int key = key0 + r;
      const bool valid = key < kv_end;
      int page = 0;
      if (valid) {
        if (TL_DEBUG_OK(key / a.page_size < a.table_width, TL_DEBUG_POSITION, key)) page = table[key / a.page_size];
        if (!TL_DEBUG_OK(page >= 0 && page < a.num_pages, TL_DEBUG_PAGE, page)) page = 0;
      }
      const __nv_bfloat16* src = a.pages + ((size_t)page * a.page_size + (valid ? key % a.page_size : 0)) * a.dk + c * 8;
      copy16(Ks + (size_t)r * stride + c * 8, src, valid);
    }
    copies_done();
    __syncthreads();

    // S for rows of rw and keys [cw KW, (cw + 1) KW)
    float s[SNT][4];
#pragma unroll
    for (int i = 0; i < SNT; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    for (int k0 = 0; k0 < (warp_has_rows ? a.dk : 0); k0 += 16) {
      unsigned qa[4];
      load_frag(qa, Qs + (size_t)(rw * 16 + (lane & 15)) * stride + k0 + (lane >> 4) * 8);
#pragma unroll
      for (int np = 0; np < SNT / 2; ++np) {
        unsigned kb[4];
        const int mi = lane >> 3;
        load_frag(kb, Ks + (size_t)(cw * KW + np * 16 + (mi >> 1) * 8 + (lane & 7)) * stride + k0 + (mi & 1) * 8);
        mma(s[2 * np], qa, kb[0], kb[1]);
        mma(s[2 * np + 1], qa, kb[2], kb[3]);
      }
    }
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int i = 0; i < SNT; ++i) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int key = key0 + cw * KW + i * 8 + t4 * 2 + j;
        s[i][j] = (on_lo && key <= pos_lo) ? s[i][j] * a.scale : -INFINITY;
        s[i][2 + j] = (on_hi && key <= pos_hi) ? s[i][2 + j] * a.scale : -INFINITY;
        mx_lo = fmaxf(mx_lo, s[i][j]);
        mx_hi = fmaxf(mx_hi, s[i][2 + j]);
      }
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    if (NCW > 1) {
      if (t4 == 0) {
        red_max[cw * ROWS + r_lo] = mx_lo;
        red_max[cw * ROWS + r_hi] = mx_hi;
      }
      __syncthreads();
#pragma unroll
      for (int c = 0; c < NCW; ++c) {
        mx_lo = fmaxf(mx_lo, red_max[c * ROWS + r_lo]);
        mx_hi = fmaxf(mx_hi, red_max[c * ROWS + r_hi]);
      }
    }
    const float new_lo = fmaxf(m_run[0], mx_lo), new_hi = fmaxf(m_run[1], mx_hi);
    const float corr_lo = new_lo == -INFINITY ? 1.f : expf(m_run[0] - new_lo);
    const float corr_hi = new_hi == -INFINITY ? 1.f : expf(m_run[1] - new_hi);
    float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
    for (int i = 0; i < SNT; ++i) {
      float p[4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        p[j] = new_lo == -INFINITY ? 0.f : expf(s[i][j] - new_lo);
        p[2 + j] = new_hi == -INFINITY ? 0.f : expf(s[i][2 + j] - new_hi);
      }
      // the sums take what the product will see: P rounded to bfloat16
      const __nv_bfloat162 lo = __floats2bfloat162_rn(p[0], p[1]), hi = __floats2bfloat162_rn(p[2], p[3]);
      sum_lo += __bfloat162float(lo.x) + __bfloat162float(lo.y);
      sum_hi += __bfloat162float(hi.x) + __bfloat162float(hi.y);
      const int col = cw * KW + i * 8 + t4 * 2;
      *reinterpret_cast<__nv_bfloat162*>(Ps + r_lo * P_STRIDE + col) = lo;
      *reinterpret_cast<__nv_bfloat162*>(Ps + r_hi * P_STRIDE + col) = hi;
    }
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
    if (NCW > 1) {
      if (t4 == 0) {
        red_sum[cw * ROWS + r_lo] = sum_lo;
        red_sum[cw * ROWS + r_hi] = sum_hi;
      }
      __syncthreads();  // also: all of P is written
      sum_lo = sum_hi = 0.f;
#pragma unroll
      for (int c = 0; c < NCW; ++c) {
        sum_lo += red_sum[c * ROWS + r_lo];
        sum_hi += red_sum[c * ROWS + r_hi];
      }
    } else {
      __syncwarp();  // a warp reads only the rows of P that it wrote itself
    }
    l_run[0] = l_run[0] * corr_lo + sum_lo;
    l_run[1] = l_run[1] * corr_hi + sum_hi;
    m_run[0] = new_lo;
    m_run[1] = new_hi;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      o[i][0] *= corr_lo;
      o[i][1] *= corr_lo;
      o[i][2] *= corr_hi;
      o[i][3] *= corr_hi;
    }
    // O += P V over the tile's 64 keys
#pragma unroll
    for (int k0 = 0; k0 < KEYS; k0 += 16) {
      if (!warp_has_rows) break;
      unsigned pa[4];
      load_frag(pa, Ps + (rw * 16 + (lane & 15)) * P_STRIDE + k0 + (lane >> 4) * 8);
#pragma unroll
      for (int np = 0; np < 8; ++np) {
        if (2 * np < nt_cnt) {
          unsigned vb[4];
          const int mi = lane >> 3;
          load_frag_t(vb, Ks + (size_t)(k0 + (mi & 1) * 8 + (lane & 7)) * stride + (nt_lo + 2 * np + (mi >> 1)) * 8);
          mma(o[2 * np], pa, vb[0], vb[1]);
          mma(o[2 * np + 1], pa, vb[2], vb[3]);
        }
      }
    }
  }

  copies_done();  // (a split without key tiles has not waited for its query rows yet)
  // results: rows r_lo and r_hi, columns (nt_lo + i) 8 + 2 t4 + {0, 1}
  const size_t grow_lo = q_row0 + r_lo, grow_hi = q_row0 + r_hi;
  if (a.splits == 1) {
    const float inv_lo = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, inv_hi = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if (i < nt_cnt) {
        const int col = (nt_lo + i) * 8 + t4 * 2;
        if (on_lo)
          *reinterpret_cast<__nv_bfloat162*>(a.out + grow_lo * a.dv + col) = __floats2bfloat162_rn(o[i][0] * inv_lo, o[i][1] * inv_lo);
        if (on_hi)
          *reinterpret_cast<__nv_bfloat162*>(a.out + grow_hi * a.dv + col) = __floats2bfloat162_rn(o[i][2] * inv_hi, o[i][3] * inv_hi);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if (i < nt_cnt) {
        const int col = (nt_lo + i) * 8 + t4 * 2;
        if (on_lo)
          *reinterpret_cast<float2*>(a.part_o + (grow_lo * a.splits + split) * a.dv + col) = make_float2(o[i][0], o[i][1]);
        if (on_hi)
          *reinterpret_cast<float2*>(a.part_o + (grow_hi * a.splits + split) * a.dv + col) = make_float2(o[i][2], o[i][3]);
      }
    }
    if (cw == 0 && t4 == 0) {
      if (on_lo) *reinterpret_cast<float2*>(a.part_ml + (grow_lo * a.splits + split) * 2) = make_float2(m_run[0], l_run[0]);
      if (on_hi) *reinterpret_cast<float2*>(a.part_ml + (grow_hi * a.splits + split) * 2) = make_float2(m_run[1], l_run[1]);
    }
  }
}

// One block per packed row: out = sum_s e^(m_s - M) O_s / sum_s e^(m_s - M) l_s.  The splits' weights
// are taken once (a thread a split), the columns run over the threads.
constexpr int MAX_SPLITS = 64;

__global__ void __launch_bounds__(128)
latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out,
                    int splits, int dv) {
  tl::pdl_wait();
  tl::pdl_launch_dependents();
  __shared__ float weight[MAX_SPLITS];
  __shared__ float inv_l;
  const size_t row = blockIdx.x;
  const float* ml = part_ml + row * splits * 2;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float m0 = lane < splits ? ml[2 * lane] : -INFINITY, m1 = lane + 32 < splits ? ml[2 * (lane + 32)] : -INFINITY;
    const float M = warp_max(fmaxf(m0, m1));
    const float w0 = m0 == -INFINITY ? 0.f : expf(m0 - M), w1 = m1 == -INFINITY ? 0.f : expf(m1 - M);
    if (lane < splits) weight[lane] = w0;
    if (lane + 32 < splits) weight[lane + 32] = w1;
    const float l = warp_sum((lane < splits ? w0 * ml[2 * lane + 1] : 0.f) +
                             (lane + 32 < splits ? w1 * ml[2 * (lane + 32) + 1] : 0.f));
    if (lane == 0) inv_l = l > 0.f ? 1.f / l : 0.f;
  }
  __syncthreads();
  const float* po = part_o + row * splits * dv;
  for (int c = threadIdx.x; c < dv; c += 128) {
    float acc = 0.f;
#pragma unroll 4
    for (int s = 0; s < splits; ++s) acc = fmaf(weight[s], po[(size_t)s * dv + c], acc);
    out[row * dv + c] = __float2bfloat16_rn(acc * inv_l);
  }
}

size_t smem_bytes(int dk, int ncw) {
  return (size_t)(ROWS + KEYS) * (dk + PAD) * 2 + (size_t)ROWS * P_STRIDE * 2 + (size_t)2 * ncw * ROWS * 4;
}

}  // namespace

TL_DEBUG_READER(tl_latent_attention_mma_debug_error)

extern "C" {

// 1 if the sizes run on this kernel.
int tl_latent_attention_mma_supported(int dk, int dv) {
  return dk % 16 == 0 && dv % 16 == 0 && dv >= 16 && dv <= 512 && dv <= dk && dk <= 640 ? 1 : 0;
}

// tiles: row tiles of the step; tile_req/tile_row null: every request brings one token and has
// tiles_per_req = ceil(heads / 64) tiles.  splits > 1 needs part_o [T heads, splits, dv] and
// part_ml [T heads, splits, 2] (float32) and launches the merge behind the product.
int tl_latent_attention_mma(const void* q, const void* pages, const int* block_table, int table_width,
                            const int* req_indptr, const int* kv_before, const int* tile_req, const int* tile_row,
                            int tiles, void* out, int tokens, int heads, int dk, int dv, int page_size, float scale,
                            int num_pages, int splits, float* part_o, float* part_ml, cudaStream_t stream) {
  if (tiles <= 0) return 0;
  if (!tl_latent_attention_mma_supported(dk, dv) || splits < 1 || splits > MAX_SPLITS) return TL_ERR_UNSUPPORTED;
  if (splits > 1 && (!part_o || !part_ml || tile_req)) return TL_ERR_UNSUPPORTED;
  Args a;
  a.q = (const __nv_bfloat16*)q;
  a.pages = (const __nv_bfloat16*)pages;
  a.block_table = block_table;
  a.req_indptr = req_indptr;
  a.kv_before = kv_before;
  a.tile_req = tile_req;
  a.tile_row = tile_row;
  a.out = (__nv_bfloat16*)out;
  a.part_o = part_o;
  a.part_ml = part_ml;
  a.table_width = table_width;
  a.heads = heads;
  a.dk = dk;
  a.dv = dv;
  a.page_size = page_size;
  a.num_pages = num_pages;
  a.tiles_per_req = (heads + ROWS - 1) / ROWS;
  a.splits = splits;
  a.scale = scale;
  const int ncw = dv <= 128 ? 1 : (dv <= 256 ? 2 : 4);
  const size_t smem = smem_bytes(dk, ncw);
  dim3 grid(tiles, splits);
  cudaError_t err;
#define TL_LAUNCH_NCW(N)                                                                                         \
  err = cudaFuncSetAttribute(latent_attention_mma_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
  if (err != cudaSuccess) return (int)err;                                                                       \
  tl::launch_kernel(latent_attention_mma_kernel<N>, grid, 128 * N, smem, stream, a)
  if (ncw == 1) { TL_LAUNCH_NCW(1); }
  else if (ncw == 2) { TL_LAUNCH_NCW(2); }
  else { TL_LAUNCH_NCW(4); }
#undef TL_LAUNCH_NCW
  int code = TL_LAUNCH_CHECK();
  if (code || splits == 1) return code;
  const long long rows = (long long)tokens * heads;
  tl::launch_kernel(latent_merge_kernel, (unsigned)rows, 128, 0, stream, (const float*)part_o,
                    (const float*)part_ml, (__nv_bfloat16*)out, splits, dv);
  return TL_LAUNCH_CHECK();
}

}  // extern "C"
