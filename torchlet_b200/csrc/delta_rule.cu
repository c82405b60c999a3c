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
//   prepare  one block per (token, head): w, u and a * u of every key channel;
//   scan     one WARP per (request, head, 32 value channels): the columns of S are independent
//            of one another, so a lane keeps one column (D floats) in registers and walks the
//            request's tokens of this step in order; r, k, v, w, u, a*u of a few tokens at a time
//            are staged in shared memory (two stages, asynchronous copies) and read as broadcasts.  The state row of the
//            request's slot is read at the start and written back at the end, so a prompt
//            cut into portions, or decoded token by token, runs the same additions in the
//            same order as the whole prompt;
//   finish   one warp per (token, head): o / rms(o) * weight * sigmoid(g) in the compute type.
#include <math.h>

#include "common.cuh"

namespace {

using namespace tl;

constexpr float DECAY_RATE = 0.6065306597126334f;  // exp(-1/2)

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }

template <int NT>
__global__ void __launch_bounds__(NT)
delta_prepare_kernel(const float* __restrict__ proj, int proj_stride, const float* __restrict__ w2,
                     const float* __restrict__ w0, const float* __restrict__ a_bias, float* __restrict__ gates,
                     int heads, int dim, int rank) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  extern __shared__ float lowrank[];  // tanh(l), rank floats
  __shared__ float scratch[32];
  const int t = blockIdx.x, h = blockIdx.y, i = threadIdx.x;
  const int hd = heads * dim;
  const float* row = proj + (size_t)t * proj_stride;
  for (int j = threadIdx.x; j < rank; j += NT) lowrank[j] = tanhf(row[5 * hd + j]);
  __syncthreads();
  const bool on = i < dim;
  const int c = h * dim + (on ? i : 0);
  const float k = on ? row[hd + c] : 0.f;
  const float ss = block_sum<NT>(k * k, scratch);
  if (!on) return;
  float inner = w0[c];
  const float* w2row = w2 + (size_t)c * rank;
  for (int j = 0; j < rank; ++j) inner = fmaf(w2row[j], lowrank[j], inner);
  const float w = expf(-DECAY_RATE * sigmoidf_(inner));
  const float a = sigmoidf_(row[4 * hd + c] + a_bias[c]);
  const float u = k / sqrtf(ss + 1e-6f);
  float* out = gates + ((size_t)t * heads + h) * 3 * dim;
  out[i] = w;
  out[dim + i] = u;
  out[2 * dim + i] = a * u;
}

__device__ __forceinline__ void copy16(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copies_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// r, k, v, w, u, a*u of CHUNK tokens are staged in shared memory, two stages deep: while the warp
// walks one chunk, the next one is on its way (16-byte asynchronous copies where D and the row
// stride are multiples of 4 floats, plain loads otherwise).
template <int DK, bool VEC>
__global__ void __launch_bounds__(32)
delta_scan_kernel(const float* __restrict__ proj, int proj_stride, const float* __restrict__ gates,
                  const int* __restrict__ req_indptr, const int* __restrict__ slots, float* __restrict__ state,
                  float* __restrict__ out, int heads, int dim, int max_slots) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  constexpr int CHUNK = DK <= 64 ? 8 : (DK <= 128 ? 4 : 2);
  __shared__ __align__(16) float stage[2][CHUNK][6][DK];  // r, k, v, w, u, a*u
  const int req = blockIdx.x, h = blockIdx.y, lane = threadIdx.x;
  const int j = blockIdx.z * 32 + lane;
  const bool on = j < dim;
  const int hd = heads * dim;
  const int first = req_indptr[req], last = req_indptr[req + 1];
  const int slot = slots[req];
  const bool live = TL_DEBUG_OK(slot >= -1 && slot < max_slots, TL_DEBUG_SLOT, slot) && slot >= 0;
  if (!live) {  // a padding lane of a captured step: no state is touched
    if (on)
      for (int t = first; t < last; ++t) out[(size_t)t * hd + h * dim + j] = 0.f;
    return;
  }
  if (!VEC || dim < DK) {  // entries past dim stay zero in both stages
    for (int e = lane; e < 2 * CHUNK * 6 * DK; e += 32) (&stage[0][0][0][0])[e] = 0.f;
    __syncwarp();
  }
  auto fetch = [&](int base, int buf) {
    const int count = last - base < CHUNK ? last - base : CHUNK;
    if (VEC) {
      const int quads = dim >> 2;
      for (int e = lane; e < count * 6 * quads; e += 32) {
        const int tt = e / (6 * quads), rest = e - tt * 6 * quads, what = rest / quads, q = rest - what * quads;
        const int t = base + tt;
        const float* src = what < 3 ? proj + (size_t)t * proj_stride + what * hd + h * dim
                                    : gates + (((size_t)t * heads + h) * 3 + (what - 3)) * dim;
        copy16(&stage[buf][tt][what][4 * q], src + 4 * q);
      }
    } else {
      for (int e = lane; e < count * 6 * dim; e += 32) {
        const int tt = e / (6 * dim), rest = e - tt * 6 * dim, what = rest / dim, i = rest - what * dim;
        const int t = base + tt;
        stage[buf][tt][what][i] = what < 3 ? proj[(size_t)t * proj_stride + what * hd + h * dim + i]
                                           : gates[(((size_t)t * heads + h) * 3 + (what - 3)) * dim + i];
      }
    }
    copies_commit();
  };
  if (first < last) fetch(first, 0);

  float* mine = state + ((size_t)slot * heads + h) * dim * dim;
  float S[DK];
#pragma unroll
  for (int i = 0; i < DK; ++i) S[i] = (on && i < dim) ? mine[(size_t)i * dim + j] : 0.f;

  int buf = 0;
  for (int base = first; base < last; base += CHUNK, buf ^= 1) {
    const int count = last - base < CHUNK ? last - base : CHUNK;
    if (base + CHUNK < last) {
      fetch(base + CHUNK, buf ^ 1);
      copies_wait<1>();
    } else {
      copies_wait<0>();
    }
    __syncwarp();
    for (int tt = 0; tt < count; ++tt) {
      const int t = base + tt;
      const float v = on ? stage[buf][tt][2][j & (DK - 1)] : 0.f;
      const float4* r4 = reinterpret_cast<const float4*>(stage[buf][tt][0]);
      const float4* k4 = reinterpret_cast<const float4*>(stage[buf][tt][1]);
      const float4* w4 = reinterpret_cast<const float4*>(stage[buf][tt][3]);
      const float4* u4 = reinterpret_cast<const float4*>(stage[buf][tt][4]);
      const float4* au4 = reinterpret_cast<const float4*>(stage[buf][tt][5]);
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;  // u^T S_old over key channels i = 0, 1, 2, 3 mod 4
#pragma unroll
      for (int q = 0; q < DK / 4; ++q) {
        const float4 u = u4[q];
        s0 = fmaf(u.x, S[4 * q], s0);
        s1 = fmaf(u.y, S[4 * q + 1], s1);
        s2 = fmaf(u.z, S[4 * q + 2], s2);
        s3 = fmaf(u.w, S[4 * q + 3], s3);
      }
      const float seen = (s0 + s1) + (s2 + s3);
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
      for (int q = 0; q < DK / 4; ++q) {
        const float4 w = w4[q], au = au4[q], k = k4[q], r = r4[q];
        S[4 * q] = fmaf(k.x, v, fmaf(-au.x, seen, w.x * S[4 * q]));
        S[4 * q + 1] = fmaf(k.y, v, fmaf(-au.y, seen, w.y * S[4 * q + 1]));
        S[4 * q + 2] = fmaf(k.z, v, fmaf(-au.z, seen, w.z * S[4 * q + 2]));
        S[4 * q + 3] = fmaf(k.w, v, fmaf(-au.w, seen, w.w * S[4 * q + 3]));
        o0 = fmaf(r.x, S[4 * q], o0);
        o1 = fmaf(r.y, S[4 * q + 1], o1);
        o2 = fmaf(r.z, S[4 * q + 2], o2);
        o3 = fmaf(r.w, S[4 * q + 3], o3);
      }
      if (on) out[(size_t)t * hd + h * dim + j] = (o0 + o1) + (o2 + o3);
    }
    __syncwarp();  // the stage is free for the chunk after the next
  }
  if (on) {
#pragma unroll
    for (int i = 0; i < DK; ++i)
      if (i < dim) mine[(size_t)i * dim + j] = S[i];
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

// gates: float32 [tokens, heads, 3, dim] scratch.
int tl_delta_prepare(const float* proj, int proj_stride, const float* w2, const float* w0, const float* a_bias,
                     float* gates, int tokens, int heads, int dim, int rank, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (dim <= 0 || dim > 1024 || heads > 65535 || rank <= 0 || rank > 8192) return TL_ERR_UNSUPPORTED;
  dim3 grid(tokens, heads);
  const size_t smem = (size_t)rank * sizeof(float);
  if (dim <= 64)
    tl::launch_kernel(delta_prepare_kernel<64>, grid, 64, smem, stream, proj, proj_stride, w2, w0, a_bias, gates, heads, dim, rank);
  else if (dim <= 128)
    tl::launch_kernel(delta_prepare_kernel<128>, grid, 128, smem, stream, proj, proj_stride, w2, w0, a_bias, gates, heads, dim, rank);
  else if (dim <= 256)
    tl::launch_kernel(delta_prepare_kernel<256>, grid, 256, smem, stream, proj, proj_stride, w2, w0, a_bias, gates, heads, dim, rank);
  else
    tl::launch_kernel(delta_prepare_kernel<1024>, grid, 1024, smem, stream, proj, proj_stride, w2, w0, a_bias, gates, heads, dim, rank);
  return TL_LAUNCH_CHECK();
}

// state: float32 [max_slots, heads, dim, dim]; out: float32 [tokens, heads * dim].
int tl_delta_scan(const float* proj, int proj_stride, const float* gates, const int* req_indptr, const int* slots,
                  float* state, float* out, int requests, int heads, int dim, int max_slots, cudaStream_t stream) {
  if (requests <= 0) return 0;
  if (dim <= 0 || dim > 256 || heads > 65535) return TL_ERR_UNSUPPORTED;
  dim3 grid(requests, heads, (dim + 31) / 32);
  const bool vec = dim % 4 == 0 && proj_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(proj) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(gates) & 15) == 0;
#define TL_SCAN(DK)                                                                                                \
  if (vec)                                                                                                         \
    tl::launch_kernel(delta_scan_kernel<DK, true>, grid, 32, 0, stream, proj, proj_stride, gates, req_indptr,      \
                      slots, state, out, heads, dim, max_slots);                                                   \
  else                                                                                                             \
    tl::launch_kernel(delta_scan_kernel<DK, false>, grid, 32, 0, stream, proj, proj_stride, gates, req_indptr,     \
                      slots, state, out, heads, dim, max_slots)
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
