// Residual-stream and normalisation kernels of hybrid decoders (float stream, typed GEMM operands):
// learned-position embedding, depth-weighted stream + single-gain RMS norm, part-wise gated RMS norm, column activations.
// Compiled WITHOUT fast-math: the float32 serving mode must stay within float rounding of a plain evaluation.
#include <cuda_bf16.h>

#include <cstdint>

#include "hybrid_kernels.h"

namespace {

__device__ __forceinline__ float ld(const float* p, long i) { return p[i]; }
__device__ __forceinline__ float ld(const __nv_bfloat16* p, long i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void st(float* p, long i, float v) { p[i] = v; }
__device__ __forceinline__ void st(__nv_bfloat16* p, long i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void st4(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void st4(__nv_bfloat16* p, const float (&v)[4]) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 u;
  u.x = *reinterpret_cast<const unsigned*>(&a);
  u.y = *reinterpret_cast<const unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}
// V consecutive floats (V = 1 or 4; 4 needs 16-byte alignment)
template <int V>
__device__ __forceinline__ void ldv(const float* p, float (&v)[V]) {
  if constexpr (V == 4) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  } else {
    v[0] = p[0];
  }
}
template <int V, typename OT>
__device__ __forceinline__ void stv(OT* p, const float (&v)[V]) {
  if constexpr (V == 4) st4(p, v);
  else st(p, 0, v[0]);
}

// sum over the block; every thread gets the result.  red: >= 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}

template <typename WT>
__global__ void embed_pos_kernel(const WT* __restrict__ embed, const WT* __restrict__ ptab, const int* __restrict__ tok,
                                 const int* __restrict__ pos, float* __restrict__ out, int W) {
  const long t = blockIdx.x;
  const long a = static_cast<long>(tok[t]) * W, b = static_cast<long>(pos[t]) * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) out[t * W + c] = ld(embed, a + c) + ld(ptab, b + c);
}

template <typename HT, int V>        // V columns per thread and pass (4: 128-bit accesses, needs W % 4 == 0)
__global__ void stream_norm_kernel(float* __restrict__ results, long stride_r, int i, const float* __restrict__ o,
                                   const float* __restrict__ xprev, const float* __restrict__ dw, const float* __restrict__ g,
                                   float eps, float* __restrict__ xcur, HT* __restrict__ h, int W) {
  __shared__ float red[32];
  const long row = static_cast<long>(blockIdx.x) * W;
  float ss = 0.f;
  for (int c = threadIdx.x * V; c < W; c += blockDim.x * V) {
    float last[V], x[V];
    if (o != nullptr) {
      float a[V], b[V];
      ldv<V>(xprev + row + c, a);
      ldv<V>(o + row + c, b);
#pragma unroll
      for (int k = 0; k < V; ++k) last[k] = a[k] + b[k];
      stv<V>(results + i * stride_r + row + c, last);
    } else {
      ldv<V>(results + i * stride_r + row + c, last);
    }
    if (dw != nullptr) {
#pragma unroll
      for (int k = 0; k < V; ++k) x[k] = 0.f;
      for (int j = 0; j < i; ++j) {
        float r[V];
        ldv<V>(results + j * stride_r + row + c, r);
        const float wj = dw[j];
#pragma unroll
        for (int k = 0; k < V; ++k) x[k] += wj * r[k];
      }
      const float wi = dw[i];
#pragma unroll
      for (int k = 0; k < V; ++k) x[k] += wi * last[k];
    } else {
#pragma unroll
      for (int k = 0; k < V; ++k) x[k] = last[k];
    }
    stv<V>(xcur + row + c, x);
#pragma unroll
    for (int k = 0; k < V; ++k) ss += x[k] * x[k];
  }
  ss = block_sum(ss, red);
  const float r = g[0] / sqrtf(ss / static_cast<float>(W) + eps);
  for (int c = threadIdx.x * V; c < W; c += blockDim.x * V) {
    float x[V];
    ldv<V>(xcur + row + c, x);
#pragma unroll
    for (int k = 0; k < V; ++k) x[k] *= r;
    stv<V>(h + row + c, x);
  }
}

template <typename OT>
__global__ void act_cols_kernel(const float* __restrict__ in, long si, OT* __restrict__ out, long so, int act, long T, int C) {
  const long n = T * C;
  for (long idx = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; idx < n; idx += static_cast<long>(gridDim.x) * blockDim.x) {
    const long t = idx / C;
    const int c = static_cast<int>(idx - t * C);
    float v = in[t * si + c];
    if (act == 1) {
      v = fmaxf(v, 0.f);
      v = v * v;
    }
    st(out, t * so + c, v);
  }
}

// four columns per thread: 128-bit loads, 64- / 128-bit stores
template <typename OT>
__global__ void act_cols_vec4_kernel(const float* __restrict__ in, long si, OT* __restrict__ out, long so, int act, long T, int C4) {
  const long n = T * C4;
  for (long idx = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; idx < n; idx += static_cast<long>(gridDim.x) * blockDim.x) {
    const long t = idx / C4;
    const int c = static_cast<int>(idx - t * C4) * 4;
    float v[4];
    ldv<4>(in + t * si + c, v);
    if (act == 1) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[i] = fmaxf(v[i], 0.f);
        v[i] = v[i] * v[i];
      }
    }
    st4(out + t * so + c, v);
  }
}

__device__ __forceinline__ float gate_fn(float z, int act) {
  const float sg = 1.f / (1.f + expf(-z));
  return act == 0 ? z * sg : sg;
}

// one warp per (token, part); V columns per lane and pass
template <typename OT, int V>
__global__ void gated_part_rmsnorm_kernel(const float* __restrict__ y, long sy, const float* __restrict__ gate, long sg,
                                          const float* __restrict__ w, int shared_w, int part, int gate_act, int gate_first,
                                          float eps, float scale, OT* __restrict__ out, long so, long T, int nparts) {
  const long wid = (blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= T * nparts) return;
  const long t = wid / nparts;
  const int p = static_cast<int>(wid - t * nparts);
  const float* yr = y + t * sy + static_cast<long>(p) * part;
  const float* gr = gate + t * sg + static_cast<long>(p) * part;
  float ss = 0.f;
  for (int c = lane * V; c < part; c += 32 * V) {
    float v[V], gv[V];
    ldv<V>(yr + c, v);
    if (gate_first) ldv<V>(gr + c, gv);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      if (gate_first) v[i] *= gate_fn(gv[i], gate_act);
      ss += v[i] * v[i];
    }
  }
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / static_cast<float>(part) + eps);
  for (int c = lane * V; c < part; c += 32 * V) {
    float v[V], gv[V], wv[V];
    ldv<V>(yr + c, v);
    ldv<V>(gr + c, gv);
    ldv<V>(w + (shared_w ? c : p * part + c), wv);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const float gg = gate_fn(gv[i], gate_act);
      v[i] = scale * (gate_first ? (v[i] * gg) * r * wv[i] : v[i] * r * wv[i] * gg);
    }
    stv<V>(out + t * so + static_cast<long>(p) * part + c, v);
  }
}

// one block per (token, part): wide parts (a warp alone would walk them serially)
template <typename OT, int V>
__global__ void gated_part_rmsnorm_block_kernel(const float* __restrict__ y, long sy, const float* __restrict__ gate, long sg,
                                                const float* __restrict__ w, int shared_w, int part, int gate_act, int gate_first,
                                                float eps, float scale, OT* __restrict__ out, long so, int nparts) {
  __shared__ float red[8];
  const long t = blockIdx.x / nparts;
  const int p = static_cast<int>(blockIdx.x - t * nparts);
  const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const float* yr = y + t * sy + static_cast<long>(p) * part;
  const float* gr = gate + t * sg + static_cast<long>(p) * part;
  float ss = 0.f;
  for (int c = threadIdx.x * V; c < part; c += blockDim.x * V) {
    float v[V], gv[V];
    ldv<V>(yr + c, v);
    if (gate_first) ldv<V>(gr + c, gv);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      if (gate_first) v[i] *= gate_fn(gv[i], gate_act);
      ss += v[i] * v[i];
    }
  }
  ss = warp_sum(ss);
  if (lane == 0) red[wi] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < nw; ++i) tot += red[i];
  const float r = 1.f / sqrtf(tot / static_cast<float>(part) + eps);
  for (int c = threadIdx.x * V; c < part; c += blockDim.x * V) {
    float v[V], gv[V], wv[V];
    ldv<V>(yr + c, v);
    ldv<V>(gr + c, gv);
    ldv<V>(w + (shared_w ? c : p * part + c), wv);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const float gg = gate_fn(gv[i], gate_act);
      v[i] = scale * (gate_first ? (v[i] * gg) * r * wv[i] : v[i] * r * wv[i] * gg);
    }
    stv<V>(out + t * so + static_cast<long>(p) * part + c, v);
  }
}

}  // namespace

namespace {
template <typename OT, int V>
cudaError_t launch_gated_norm(const float* y, long sy, const float* gate, long sg, const float* w, int shared_w, int part, int gate_act,
                              int gate_first, float eps, float scale, OT* out, long so, int T, int nparts, cudaStream_t s) {
  const long warps = static_cast<long>(T) * nparts;
  if (part >= 256) {
    const int th = part >= 1024 * V / 4 ? 256 : 128;
    gated_part_rmsnorm_block_kernel<OT, V><<<static_cast<unsigned>(warps), th, 0, s>>>(y, sy, gate, sg, w, shared_w, part, gate_act,
                                                                                      gate_first, eps, scale, out, so, nparts);
  } else {
    gated_part_rmsnorm_kernel<OT, V><<<static_cast<unsigned>((warps + 3) / 4), 128, 0, s>>>(y, sy, gate, sg, w, shared_w, part, gate_act,
                                                                                            gate_first, eps, scale, out, so, T, nparts);
  }
  return cudaGetLastError();
}
}  // namespace

namespace {
inline bool aligned(const void* p, size_t a) { return reinterpret_cast<uintptr_t>(p) % a == 0; }
}  // namespace

extern "C" {

cudaError_t nrl_embed_pos(const void* embed, const void* pos_table, int w_f32, const int* tok, const int* pos, float* out, int T,
                          int W, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  const int th = W >= 256 ? 256 : 128;
  if (w_f32)
    embed_pos_kernel<float><<<T, th, 0, s>>>(static_cast<const float*>(embed), static_cast<const float*>(pos_table), tok, pos, out, W);
  else
    embed_pos_kernel<__nv_bfloat16><<<T, th, 0, s>>>(static_cast<const __nv_bfloat16*>(embed),
                                                    static_cast<const __nv_bfloat16*>(pos_table), tok, pos, out, W);
  return cudaGetLastError();
}

cudaError_t nrl_stream_norm(float* results, long stride_r, int i, const float* o, const float* xprev, const float* dw,
                            const float* g, float eps, float* xcur, void* h, int h_f32, int T, int W, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  const bool vec = W % 4 == 0 && stride_r % 4 == 0 && aligned(results, 16) && aligned(xcur, 16) && aligned(h, h_f32 ? 16 : 8) &&
                   (o == nullptr || (aligned(o, 16) && aligned(xprev, 16)));
  const int th = W >= 1024 * (vec ? 4 : 1) ? 256 : 128;
#define NRL_SN(HT_, V_)                                                                                                            \
  stream_norm_kernel<HT_, V_><<<T, th, 0, s>>>(results, stride_r, i, o, xprev, dw, g, eps, xcur, static_cast<HT_*>(h), W)
  if (h_f32) {
    if (vec) NRL_SN(float, 4);
    else NRL_SN(float, 1);
  } else {
    if (vec) NRL_SN(__nv_bfloat16, 4);
    else NRL_SN(__nv_bfloat16, 1);
  }
#undef NRL_SN
  return cudaGetLastError();
}

cudaError_t nrl_act_cols(const float* in, long si, void* out, long so, int out_f32, int act, int T, int C, cudaStream_t s) {
  if (T <= 0 || C <= 0) return cudaSuccess;
  const size_t out_align = out_f32 ? 16 : 8;
  if (C % 4 == 0 && si % 4 == 0 && so % 4 == 0 && aligned(in, 16) && aligned(out, out_align)) {
    const long n = static_cast<long>(T) * (C / 4);
    const int blocks = static_cast<int>((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    if (out_f32)
      act_cols_vec4_kernel<float><<<blocks, 256, 0, s>>>(in, si, static_cast<float*>(out), so, act, T, C / 4);
    else
      act_cols_vec4_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(in, si, static_cast<__nv_bfloat16*>(out), so, act, T, C / 4);
    return cudaGetLastError();
  }
  const long n = static_cast<long>(T) * C;
  const int blocks = static_cast<int>((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  if (out_f32)
    act_cols_kernel<float><<<blocks, 256, 0, s>>>(in, si, static_cast<float*>(out), so, act, T, C);
  else
    act_cols_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(in, si, static_cast<__nv_bfloat16*>(out), so, act, T, C);
  return cudaGetLastError();
}

cudaError_t nrl_gated_part_rmsnorm(const float* y, long sy, const float* gate, long sg, const float* w, int shared_w, int part,
                                   int gate_act, int gate_first, float eps, float scale, void* out, long so, int out_f32, int T,
                                   int n, cudaStream_t s) {
  if (T <= 0 || n <= 0) return cudaSuccess;
  if (part <= 0 || n % part != 0) return cudaErrorInvalidValue;
  const int nparts = n / part;
  const bool vec = part % 4 == 0 && sy % 4 == 0 && sg % 4 == 0 && so % 4 == 0 && aligned(y, 16) && aligned(gate, 16) && aligned(w, 16) &&
                   aligned(out, out_f32 ? 16 : 8);
#define NRL_GN(OT_, V_)                                                                                                            \
  return launch_gated_norm<OT_, V_>(y, sy, gate, sg, w, shared_w, part, gate_act, gate_first, eps, scale, static_cast<OT_*>(out), so, T, \
                                    nparts, s)
  if (out_f32) {
    if (vec) NRL_GN(float, 4);
    NRL_GN(float, 1);
  }
  if (vec) NRL_GN(__nv_bfloat16, 4);
  NRL_GN(__nv_bfloat16, 1);
#undef NRL_GN
}

}  // extern "C"
