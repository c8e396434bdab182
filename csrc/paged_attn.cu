// Ragged attention over a paged KV cache, with optional attention sinks and an optional sliding window.
//
// A serving step is a flat list of query tokens: token t belongs to the sequence in cache row `slot[t]` and sits at
// position `pos[t]` of it. A prompt piece contributes consecutive positions, a decoding sequence one token, and the two
// kinds share a launch. The cache is [blocks, Hkv, block_size, D] per layer with a block table [rows, max_blocks]
// (logical block j of a row -> physical block). The step first stores the new tokens' K/V, then every query reads keys
// 0 .. pos[t] of its own row, so a piece attends to the pieces before it and to its own earlier tokens with no special case.
//
//   b200_rope_paged_store   rotary embedding on q (in place) and k, k -> cache K; the value rows come either from a v
//                           section of the projection or (v_from_k) are the keys as projected, before rotation.
//                           Pairs are interleaved (2i, 2i+1) or split (i, i + rot/2); only the first `rot` dims turn.
//   b200_paged_attn         one warp per (token, query head): keys are walked 32 at a time (one key per lane for the
//                           scores, one output column set per lane for P V), online softmax in fp32, any head size up
//                           to 256, 16-bit or 32-bit cache. `nsplit` > 1 cuts the keys of every token into that many
//                           ranges (long-context decode) and a second kernel merges the partial (max, sum, acc) triples.
//   b200_paged_attn_mma     16-bit prompt pieces on the tensor cores (mma.sync m16n8k16): 64 query rows of one piece per
//                           CTA, one cache page (or 64 keys of it) per iteration.
//
// A sink is a per-head logit that takes part in the softmax denominator only: the running maximum starts at the sink and
// the running sum at 1, which is exp(sink - max) for that start.
#include "common.cuh"
#include "../include/b200_ops.h"

namespace b200 {

// ------------------------------------------------------------------------------------------------------------------
// rotary + cache store
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
rope_paged_store_kernel(T* __restrict__ qkv, long long row_stride, const float* __restrict__ cs, const float* __restrict__ sn,
                        const int* __restrict__ pos, const int* __restrict__ slot, const int* __restrict__ table, int max_blocks,
                        T* __restrict__ ck, T* __restrict__ cv, int H, int G, int D, int rot, int block_size, int interleaved,
                        int v_from_k) {
  const int t = blockIdx.x;
  const int p = pos[t];
  const int s = slot[t];
  T* row = qkv + (long long)t * row_stride;
  const float* c = cs + (long long)p * (rot / 2);
  const float* sgn = sn + (long long)p * (rot / 2);
  const int blk = table[(long long)s * max_blocks + p / block_size];
  const int off = p % block_size;
  const int hr = rot / 2;
  // item i < hr: the rotary pair i; item i >= hr: the pass-through dims rot + 2 (i - hr) and the one after it
  const int items = hr + (D - rot + 1) / 2;
  for (int w = threadIdx.x; w < (H + G) * items; w += blockDim.x) {
    const int h = w / items, i = w % items;
    T* x = row + (long long)h * D;
    int d0, d1;
    bool turn = i < hr;
    if (turn) {
      d0 = interleaved ? 2 * i : i;
      d1 = interleaved ? 2 * i + 1 : i + hr;
    } else {
      d0 = rot + 2 * (i - hr);
      d1 = d0 + 1;
    }
    const bool has1 = d1 < D;
    const float u = to_f32<T>(x[d0]);
    const float v = has1 ? to_f32<T>(x[d1]) : 0.f;
    float ru = u, rv = v;
    if (turn) {
      const float cc = c[i], ss = sgn[i];
      ru = u * cc - v * ss;
      rv = v * cc + u * ss;
      x[d0] = from_f32<T>(ru);
      x[d1] = from_f32<T>(rv);
    }
    if (h >= H) {
      const int g = h - H;
      const long long base = (((long long)blk * G + g) * block_size + off) * D;
      ck[base + d0] = from_f32<T>(ru);
      if (has1) ck[base + d1] = from_f32<T>(rv);
      if (v_from_k) {
        cv[base + d0] = from_f32<T>(u);
        if (has1) cv[base + d1] = from_f32<T>(v);
      }
    }
  }
  if (!v_from_k) {
    const T* vsrc = row + (long long)(H + G) * D;
    for (int w = threadIdx.x; w < G * D; w += blockDim.x) {
      const int g = w / D, d = w % D;
      cv[(((long long)blk * G + g) * block_size + off) * D + d] = vsrc[w];
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// one warp per (token, query head)
// ------------------------------------------------------------------------------------------------------------------
constexpr int kMaxD = 256;
constexpr int kAccPerLane = kMaxD / 32;

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const T* __restrict__ k, int D) {
  float acc = 0.f;
  for (int d = 0; d < D; ++d) acc = fmaf(q[d], to_f32<T>(k[d]), acc);
  return acc;
}
template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k, int D) {
  float acc = 0.f;
  if ((D & 7) == 0) {
    for (int d = 0; d < D; d += 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(k + d);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(w[j]);
        acc = fmaf(q[d + 2 * j], f.x, acc);
        acc = fmaf(q[d + 2 * j + 1], f.y, acc);
      }
    }
  } else {
    for (int d = 0; d < D; ++d) acc = fmaf(q[d], __bfloat162float(k[d]), acc);
  }
  return acc;
}

// q: [tokens, q_stride] (head h at h * D); out: [tokens, H * D]; part: [tokens, H, nsplit, D + 2] fp32 when nsplit > 1
template <typename T>
__global__ void __launch_bounds__(256)
paged_attn_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ ck, const T* __restrict__ cv,
                  const int* __restrict__ pos, const int* __restrict__ slot, const int* __restrict__ table, int max_blocks,
                  const float* __restrict__ sinks, T* __restrict__ out, float* __restrict__ part, int H, int G, int D,
                  int block_size, float scale, int window, int nsplit) {
  extern __shared__ float qs[];                      // [warps, D]
  const int t = blockIdx.x;
  const int g = blockIdx.y;
  const int split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = blockDim.x >> 5;
  const int rep = H / G;
  const int p = pos[t];
  const int s = slot[t];
  const int* trow = table + (long long)s * max_blocks;
  int k_lo = 0, k_hi = p + 1;                        // keys [k_lo, k_hi)
  if (window > 0 && p + 1 - window > 0) k_lo = p + 1 - window;
  if (nsplit > 1) {
    const int span = k_hi - k_lo;
    const int chunk = ((span + nsplit - 1) / nsplit + 31) / 32 * 32;
    k_lo = k_lo + split * chunk;
    k_hi = min(k_hi, k_lo + chunk);
  }
  float* myq = qs + warp * D;
  for (int hh = warp; hh < rep; hh += nwarps) {
    const int h = g * rep + hh;
    const T* qr = q + (long long)t * q_stride + (long long)h * D;
    __syncwarp();
    for (int d = lane; d < D; d += 32) myq[d] = to_f32<T>(qr[d]);
    __syncwarp();
    const bool own_sink = sinks != nullptr && nsplit == 1;
    float m = own_sink ? sinks[h] : -INFINITY;
    float l = own_sink ? 1.f : 0.f;
    float acc[kAccPerLane];
#pragma unroll
    for (int i = 0; i < kAccPerLane; ++i) acc[i] = 0.f;
    for (int k0 = k_lo; k0 < k_hi; k0 += 32) {
      const int kp = k0 + lane;
      const bool valid = kp < k_hi;
      long long rowoff = 0;
      float sc = -INFINITY;
      if (valid) {
        const int blk = trow[kp / block_size];
        rowoff = (((long long)blk * G + g) * block_size + kp % block_size) * D;
        sc = dot_row<T>(myq, ck + rowoff, D) * scale;
      }
      const float m_new = fmaxf(m, warp_max(sc));
      const float pj = valid ? expf(sc - m_new) : 0.f;
      const float resc = (m == -INFINITY) ? 0.f : expf(m - m_new);
      l = l * resc + warp_sum(pj);
      m = m_new;
#pragma unroll
      for (int i = 0; i < kAccPerLane; ++i) acc[i] *= resc;
      const int nk = min(32, k_hi - k0);
      for (int j = 0; j < nk; ++j) {
        const float w = __shfl_sync(0xffffffffu, pj, j);
        const long long ro = __shfl_sync(0xffffffffu, rowoff, j);
        const T* vr = cv + ro;
#pragma unroll
        for (int i = 0; i < kAccPerLane; ++i) {
          const int d = lane + 32 * i;
          if (d < D) acc[i] = fmaf(w, to_f32<T>(vr[d]), acc[i]);
        }
      }
    }
    if (nsplit == 1) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      T* orow = out + (long long)t * H * D + (long long)h * D;
#pragma unroll
      for (int i = 0; i < kAccPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < D) orow[d] = from_f32<T>(acc[i] * inv);
      }
    } else {
      float* pr = part + (((long long)t * H + h) * nsplit + split) * (D + 2);
      if (lane == 0) { pr[0] = m; pr[1] = l; }
#pragma unroll
      for (int i = 0; i < kAccPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < D) pr[2 + d] = acc[i];
      }
    }
  }
}

template <typename T>
__global__ void paged_attn_merge_kernel(const float* __restrict__ part, const float* __restrict__ sinks, T* __restrict__ out,
                                        int H, int D, int nsplit) {
  const int t = blockIdx.x, h = blockIdx.y;
  const float* pr = part + ((long long)t * H + h) * nsplit * (D + 2);
  float m = sinks ? sinks[h] : -INFINITY;
  for (int s = 0; s < nsplit; ++s) m = fmaxf(m, pr[s * (D + 2)]);
  float l = sinks ? expf(sinks[h] - m) : 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float ms = pr[s * (D + 2)];
    if (ms != -INFINITY) l += pr[s * (D + 2) + 1] * expf(ms - m);
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float ms = pr[s * (D + 2)];
      if (ms != -INFINITY) a += pr[s * (D + 2) + 2 + d] * expf(ms - m);
    }
    out[((long long)t * H + h) * D + d] = from_f32<T>(a * inv);
  }
}

}  // namespace b200

using namespace b200;

B200_API int b200_rope_paged_store(void* qkv, long long row_stride, const void* cos_t, const void* sin_t, const void* pos,
                                   const void* slot, const void* table, int max_blocks, void* ck, void* cv, int tokens, int H,
                                   int G, int D, int rot, int block_size, int interleaved, int v_from_k, int dtype, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (tokens <= 0) return 0;
  if (H < 0 || G <= 0 || D <= 0 || rot < 0 || rot > D || (rot & 1) || block_size <= 0) return B200_ERR_BAD_SHAPE;
#define ROPE_LAUNCH(T)                                                                                                        \
  rope_paged_store_kernel<T><<<tokens, 128, 0, st>>>((T*)qkv, row_stride, (const float*)cos_t, (const float*)sin_t,           \
                                                     (const int*)pos, (const int*)slot, (const int*)table, max_blocks, (T*)ck, \
                                                     (T*)cv, H, G, D, rot, block_size, interleaved, v_from_k)
  if (dtype == B200_DT_BF16) ROPE_LAUNCH(__nv_bfloat16);
  else if (dtype == B200_DT_FP16) ROPE_LAUNCH(__half);
  else if (dtype == B200_DT_FP32) ROPE_LAUNCH(float);
  else return B200_ERR_UNSUPPORTED;
#undef ROPE_LAUNCH
  B200_LAUNCH_CHECK();
  return 0;
}

B200_API int b200_paged_attn(const void* q, long long q_stride, const void* ck, const void* cv, const void* pos, const void* slot,
                             const void* table, int max_blocks, const void* sinks, void* out, void* part, int tokens, int H, int G,
                             int D, int block_size, float scale, int window, int nsplit, int dtype, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (tokens <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || D <= 0 || D > kMaxD || block_size <= 0 || nsplit < 1) return B200_ERR_BAD_SHAPE;
  if (nsplit > 1 && !part) return B200_ERR_BAD_SHAPE;
  const int rep = H / G;
  const int warps = rep < 8 ? rep : 8;
  dim3 grid(tokens, G, nsplit), block(32 * warps);
  const size_t smem = (size_t)warps * D * sizeof(float);
#define ATTN_LAUNCH(T)                                                                                                          \
  do {                                                                                                                          \
    paged_attn_kernel<T><<<grid, block, smem, st>>>((const T*)q, q_stride, (const T*)ck, (const T*)cv, (const int*)pos,         \
                                                    (const int*)slot, (const int*)table, max_blocks, (const float*)sinks,       \
                                                    (T*)out, (float*)part, H, G, D, block_size, scale, window, nsplit);         \
    if (nsplit > 1)                                                                                                             \
      paged_attn_merge_kernel<T><<<dim3(tokens, H), 64, 0, st>>>((const float*)part, (const float*)sinks, (T*)out, H, D, nsplit); \
  } while (0)
  if (dtype == B200_DT_BF16) ATTN_LAUNCH(__nv_bfloat16);
  else if (dtype == B200_DT_FP16) ATTN_LAUNCH(__half);
  else if (dtype == B200_DT_FP32) ATTN_LAUNCH(float);
  else return B200_ERR_UNSUPPORTED;
#undef ATTN_LAUNCH
  B200_LAUNCH_CHECK();
  return 0;
}
