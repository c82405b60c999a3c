// The generalized delta rule: a recurrent mixer whose per-request state is one D x D
// float32 matrix per head (key channel i, value channel j), carried from token to token:
//
//   S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T,    o_t = S_t^T r_t
//
// with u = k / sqrt(sum(k^2) + 1e-6), decay w = exp(-exp(-1/2) sigmoid(W2 tanh(l) + w0)) in
// (0.545, 1) and removal rate a = sigmoid(a' + b).  Everything here is float32, also in the
// bfloat16 engine: the projections arrive as float32 rows
//   proj[t] = [ r (H D) | k (H D) | v (H D) | g (H D) | a' (H D) | l (rank) ].
//
// Three kernels:
//   prepare  one block per (8 tokens, head): w, u and a * u of every key channel;
//   scan     one block per (request, head): the columns of S are independent of one another;
//            four lanes share a column, each keeps a quarter of it in registers (and serves two
//            columns, so that the vectors it reads are used twice), and the block
//            walks the request's tokens of this step in order; r, k, v, w, u, a*u of a few tokens
//            at a time are staged in shared memory (two stages, asynchronous copies).  The state
//            row of the request's slot is read at the start and written back at the end, so a
//            prompt cut into portions, or decoded token by token, runs the same additions in the
//            same order as the whole prompt;
//   finish   one warp per (token, head): o / rms(o) * weight * sigmoid(g) in the compute type.
#include <math.h>

#include "common.cuh"

namespace {

using namespace tl;

constexpr float DECAY_RATE = 0.6065306597126334f;  // exp(-1/2)

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }

constexpr int PREP_TOKENS = 8;  // tokens a block of the prepare kernel takes: a W2 entry is read once for all

// w2t: W2 transposed, [rank, heads * dim], so that the threads of a block read consecutive entries.
template <int NT>
__global__ void __launch_bounds__(NT)
delta_prepare_kernel(const float* __restrict__ proj, int proj_stride, const float* __restrict__ w2t,
                     const float* __restrict__ w0, const float* __restrict__ a_bias, float* __restrict__ gates,
                     int tokens, int heads, int dim, int rank) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  extern __shared__ float lowrank[];  // tanh(l): PREP_TOKENS x rank floats
  __shared__ float scratch[32];
  const int t0 = blockIdx.x * PREP_TOKENS, h = blockIdx.y, i = threadIdx.x;
  const int count = tokens - t0 < PREP_TOKENS ? tokens - t0 : PREP_TOKENS;
  const int hd = heads * dim;
  for (int e = threadIdx.x; e < PREP_TOKENS * rank; e += NT) {
    const int tt = e / rank, j = e - tt * rank;
    lowrank[e] = tt < count ? tanhf(proj[(size_t)(t0 + tt) * proj_stride + 5 * hd + j]) : 0.f;
  }
  __syncthreads();
  const bool on = i < dim;
  const int c = h * dim + (on ? i : 0);
  float inner[PREP_TOKENS];
#pragma unroll
  for (int tt = 0; tt < PREP_TOKENS; ++tt) inner[tt] = w0[c];
  if (on) {
#pragma unroll 8
    for (int j = 0; j < rank; ++j) {
      const float w = w2t[(size_t)j * hd + c];
#pragma unroll
      for (int tt = 0; tt < PREP_TOKENS; ++tt) inner[tt] = fmaf(w, lowrank[tt * rank + j], inner[tt]);
    }
  }
#pragma unroll
  for (int tt = 0; tt < PREP_TOKENS; ++tt) {
    if (tt >= count) break;  // (the same for every thread of the block)
    const float* row = proj + (size_t)(t0 + tt) * proj_stride;
    const float k = on ? row[hd + c] : 0.f;
    const float ss = block_sum<NT>(k * k, scratch);
    if (on) {
      const float w = expf(-DECAY_RATE * sigmoidf_(inner[tt]));
      const float a = sigmoidf_(row[4 * hd + c] + a_bias[c]);
      const float u = k / sqrtf(ss + 1e-6f);
      float* out = gates + ((size_t)(t0 + tt) * heads + h) * 3 * dim;
      out[i] = w;
      out[dim + i] = u;
      out[2 * dim + i] = a * u;
    }
  }
}

__device__ __forceinline__ void copy16(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copies_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// One block per (request, head).  Four lanes share a column of S (value channel j): lane part p
// keeps the key channels i with (i / 4) % 4 == p, and the two sums over i of a token (u^T S and
// S^T r) meet by two shuffles.  A lane serves CPL = 2 columns (j and j + D/2) with the same vector
// entries, so that what it reads from shared memory is used twice: the kernel is bound by the
// shared-memory wavefronts of these reads.  All warps of the block read the same staged r, k, v,
// w, u, a*u of CHUNK tokens, two stages deep: while the block walks one chunk, the next is on its
// way (16-byte asynchronous copies where D and the row stride are multiples of 4 floats, plain
// loads otherwise).
constexpr int KS = 4;
constexpr int CPL = 2;

template <int DK, bool VEC>
__global__ void __launch_bounds__(DK * KS / CPL)
delta_scan_kernel(const float* __restrict__ proj, int proj_stride, const float* __restrict__ gates,
                  const int* __restrict__ req_indptr, const int* __restrict__ slots, float* __restrict__ state,
                  float* __restrict__ out, int heads, int dim, int max_slots) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  constexpr int NT = DK * KS / CPL;
  constexpr int PER = DK / KS;  // key channels a lane keeps of each of its columns
  constexpr int CHUNK = DK <= 64 ? 8 : (DK <= 128 ? 4 : 2);
  __shared__ __align__(16) float stage[2][CHUNK][6][DK];  // r, k, v, w, u, a*u
  const int req = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int part = tid % KS;
  int col[CPL];
  bool on[CPL];
#pragma unroll
  for (int c = 0; c < CPL; ++c) {
    col[c] = tid / KS + c * (DK / CPL);
    on[c] = col[c] < dim;
  }
  const int hd = heads * dim;
  const int first = req_indptr[req], last = req_indptr[req + 1];
  const int slot = slots[req];
  const bool live = TL_DEBUG_OK(slot >= -1 && slot < max_slots, TL_DEBUG_SLOT, slot) && slot >= 0;
  if (!live) {  // a padding lane of a captured step: no state is touched
    if (part == 0)
      for (int t = first; t < last; ++t)
#pragma unroll
        for (int c = 0; c < CPL; ++c)
          if (on[c]) out[(size_t)t * hd + h * dim + col[c]] = 0.f;
    return;
  }
  if (!VEC || dim < DK) {  // entries past dim stay zero in both stages
    for (int e = tid; e < 2 * CHUNK * 6 * DK; e += NT) (&stage[0][0][0][0])[e] = 0.f;
    __syncthreads();
  }
  auto fetch = [&](int base, int buf) {
    const int count = last - base < CHUNK ? last - base : CHUNK;
    if (VEC) {
      const int quads = dim >> 2;
      for (int e = tid; e < count * 6 * quads; e += NT) {
        const int tt = e / (6 * quads), rest = e - tt * 6 * quads, what = rest / quads, q = rest - what * quads;
        const int t = base + tt;
        const float* src = what < 3 ? proj + (size_t)t * proj_stride + what * hd + h * dim
                                    : gates + (((size_t)t * heads + h) * 3 + (what - 3)) * dim;
        copy16(&stage[buf][tt][what][4 * q], src + 4 * q);
      }
    } else {
      for (int e = tid; e < count * 6 * dim; e += NT) {
        const int tt = e / (6 * dim), rest = e - tt * 6 * dim, what = rest / dim, i = rest - what * dim;
        const int t = base + tt;
        stage[buf][tt][what][i] = what < 3 ? proj[(size_t)t * proj_stride + what * hd + h * dim + i]
                                           : gates[(((size_t)t * heads + h) * 3 + (what - 3)) * dim + i];
      }
    }
    copies_commit();
  };
  if (first < last) fetch(first, 0);

  // this lane's key channels: i = 4 (q KS + part) + e, q = 0 .. PER/4 - 1, e = 0 .. 3
  float* mine = state + ((size_t)slot * heads + h) * dim * dim;
  float S[CPL][PER];
#pragma unroll
  for (int c = 0; c < CPL; ++c)
#pragma unroll
    for (int n = 0; n < PER; ++n) {
      const int i = 4 * ((n >> 2) * KS + part) + (n & 3);
      S[c][n] = (on[c] && i < dim) ? mine[(size_t)i * dim + col[c]] : 0.f;
    }

  int buf = 0;
  for (int base = first; base < last; base += CHUNK, buf ^= 1) {
    const int count = last - base < CHUNK ? last - base : CHUNK;
    if (base + CHUNK < last) {
      fetch(base + CHUNK, buf ^ 1);
      copies_wait<1>();
    } else {
      copies_wait<0>();
    }
    __syncthreads();
    for (int tt = 0; tt < count; ++tt) {
      const int t = base + tt;
      const float4* r4 = reinterpret_cast<const float4*>(stage[buf][tt][0]);
      const float4* k4 = reinterpret_cast<const float4*>(stage[buf][tt][1]);
      const float4* w4 = reinterpret_cast<const float4*>(stage[buf][tt][3]);
      const float4* u4 = reinterpret_cast<const float4*>(stage[buf][tt][4]);
      const float4* au4 = reinterpret_cast<const float4*>(stage[buf][tt][5]);
      float v[CPL], seen[CPL], o[CPL];
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        v[c] = stage[buf][tt][2][col[c] & (DK - 1)];
        seen[c] = 0.f;
        o[c] = 0.f;
      }
      float part_seen[CPL][4];
#pragma unroll
      for (int c = 0; c < CPL; ++c) part_seen[c][0] = part_seen[c][1] = part_seen[c][2] = part_seen[c][3] = 0.f;
#pragma unroll
      for (int q = 0; q < PER / 4; ++q) {
        const float4 u = u4[q * KS + part];
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
          part_seen[c][0] = fmaf(u.x, S[c][4 * q], part_seen[c][0]);
          part_seen[c][1] = fmaf(u.y, S[c][4 * q + 1], part_seen[c][1]);
          part_seen[c][2] = fmaf(u.z, S[c][4 * q + 2], part_seen[c][2]);
          part_seen[c][3] = fmaf(u.w, S[c][4 * q + 3], part_seen[c][3]);
        }
      }
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        seen[c] = (part_seen[c][0] + part_seen[c][1]) + (part_seen[c][2] + part_seen[c][3]);
        seen[c] += __shfl_xor_sync(0xffffffffu, seen[c], 1);
        seen[c] += __shfl_xor_sync(0xffffffffu, seen[c], 2);
      }
      float part_o[CPL][4];
#pragma unroll
      for (int c = 0; c < CPL; ++c) part_o[c][0] = part_o[c][1] = part_o[c][2] = part_o[c][3] = 0.f;
#pragma unroll
      for (int q = 0; q < PER / 4; ++q) {
        const float4 w = w4[q * KS + part], au = au4[q * KS + part], k = k4[q * KS + part], r = r4[q * KS + part];
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
          S[c][4 * q] = fmaf(k.x, v[c], fmaf(-au.x, seen[c], w.x * S[c][4 * q]));
          S[c][4 * q + 1] = fmaf(k.y, v[c], fmaf(-au.y, seen[c], w.y * S[c][4 * q + 1]));
          S[c][4 * q + 2] = fmaf(k.z, v[c], fmaf(-au.z, seen[c], w.z * S[c][4 * q + 2]));
          S[c][4 * q + 3] = fmaf(k.w, v[c], fmaf(-au.w, seen[c], w.w * S[c][4 * q + 3]));
          part_o[c][0] = fmaf(r.x, S[c][4 * q], part_o[c][0]);
          part_o[c][1] = fmaf(r.y, S[c][4 * q + 1], part_o[c][1]);
          part_o[c][2] = fmaf(r.z, S[c][4 * q + 2], part_o[c][2]);
          part_o[c][3] = fmaf(r.w, S[c][4 * q + 3], part_o[c][3]);
        }
      }
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        o[c] = (part_o[c][0] + part_o[c][1]) + (part_o[c][2] + part_o[c][3]);
        o[c] += __shfl_xor_sync(0xffffffffu, o[c], 1);
        o[c] += __shfl_xor_sync(0xffffffffu, o[c], 2);
        if (on[c] && part == 0) out[(size_t)t * hd + h * dim + col[c]] = o[c];
      }
    }
    __syncthreads();  // the stage is free for the chunk after the next
  }
#pragma unroll
  for (int c = 0; c < CPL; ++c)
    if (on[c]) {
#pragma unroll
      for (int n = 0; n < PER; ++n) {
        const int i = 4 * ((n >> 2) * KS + part) + (n & 3);
        if (i < dim) mine[(size_t)i * dim + col[c]] = S[c][n];
      }
    }
}

constexpr int FINISH_WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(FINISH_WARPS * 32)
delta_finish_kernel(const float* __restrict__ o, const float* __restrict__ proj, int proj_stride,
                    const float* __restrict__ weight, T* __restrict__ out, long long items, int heads, int dim,
                    float eps) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * FINISH_WARPS + warp;
  if (item >= items) return;
  const long long t = item / heads;
  const int h = (int)(item % heads);
  const int hd = heads * dim;
  const float* row = o + (size_t)t * hd + h * dim;
  float ss = 0.f;
  for (int i = lane; i < dim; i += 32) ss = fmaf(row[i], row[i], ss);
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)dim + eps);
  const float* gate = proj + (size_t)t * proj_stride + 3 * hd + h * dim;
  for (int i = lane; i < dim; i += 32)
    out[(size_t)t * hd + h * dim + i] = from_float<T>(row[i] * inv * weight[h * dim + i] * sigmoidf_(gate[i]));
}

}  // namespace

TL_DEBUG_READER(tl_delta_rule_debug_error)

extern "C" {

// gates: float32 [tokens, heads, 3, dim] scratch;  w2t: [rank, heads * dim].
int tl_delta_prepare(const float* proj, int proj_stride, const float* w2t, const float* w0, const float* a_bias,
                     float* gates, int tokens, int heads, int dim, int rank, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (dim <= 0 || dim > 1024 || heads > 65535 || rank <= 0 || rank > 1024) return TL_ERR_UNSUPPORTED;
  dim3 grid((tokens + PREP_TOKENS - 1) / PREP_TOKENS, heads);
  const size_t smem = (size_t)PREP_TOKENS * rank * sizeof(float);
#define TL_PREPARE(NT)                                                                                            \
  tl::launch_kernel(delta_prepare_kernel<NT>, grid, NT, smem, stream, proj, proj_stride, w2t, w0, a_bias, gates,  \
                    tokens, heads, dim, rank)
  if (dim <= 32) { TL_PREPARE(32); }
  else if (dim <= 64) { TL_PREPARE(64); }
  else if (dim <= 128) { TL_PREPARE(128); }
  else if (dim <= 256) { TL_PREPARE(256); }
  else { TL_PREPARE(1024); }
#undef TL_PREPARE
  return TL_LAUNCH_CHECK();
}

// state: float32 [max_slots, heads, dim, dim]; out: float32 [tokens, heads * dim].
int tl_delta_scan(const float* proj, int proj_stride, const float* gates, const int* req_indptr, const int* slots,
                  float* state, float* out, int requests, int heads, int dim, int max_slots, cudaStream_t stream) {
  if (requests <= 0) return 0;
  if (dim <= 0 || dim > 256 || heads > 65535) return TL_ERR_UNSUPPORTED;
  dim3 grid(requests, heads);
  const bool vec = dim % 4 == 0 && proj_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(proj) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(gates) & 15) == 0;
#define TL_SCAN(DK)                                                                                                \
  if (vec)                                                                                                         \
    tl::launch_kernel(delta_scan_kernel<DK, true>, grid, DK * KS / CPL, 0, stream, proj, proj_stride, gates, req_indptr, \
                      slots, state, out, heads, dim, max_slots);                                                   \
  else                                                                                                             \
    tl::launch_kernel(delta_scan_kernel<DK, false>, grid, DK * KS / CPL, 0, stream, proj, proj_stride, gates,            \
                      req_indptr, slots, state, out, heads, dim, max_slots)
  if (dim <= 16) { TL_SCAN(16); }
  else if (dim <= 32) { TL_SCAN(32); }
  else if (dim <= 64) { TL_SCAN(64); }
  else if (dim <= 128) { TL_SCAN(128); }
  else { TL_SCAN(256); }
#undef TL_SCAN
  return TL_LAUNCH_CHECK();
}

int tl_delta_finish(const float* o, const float* proj, int proj_stride, const float* weight, void* out, int out_dtype,
                    int tokens, int heads, int dim, float eps, cudaStream_t stream) {
  const long long items = (long long)tokens * heads;
  if (items <= 0) return 0;
  const unsigned blocks = (unsigned)((items + FINISH_WARPS - 1) / FINISH_WARPS);
  if (out_dtype == TL_DTYPE_F32)
    tl::launch_kernel(delta_finish_kernel<float>, blocks, FINISH_WARPS * 32, 0, stream, o, proj, proj_stride, weight,
                      (float*)out, items, heads, dim, eps);
  else
    tl::launch_kernel(delta_finish_kernel<__nv_bfloat16>, blocks, FINISH_WARPS * 32, 0, stream, o, proj, proj_stride,
                      weight, (__nv_bfloat16*)out, items, heads, dim, eps);
  return TL_LAUNCH_CHECK();
}

}  // extern "C"
