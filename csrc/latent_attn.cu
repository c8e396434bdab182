// Attention over a cache of latent rows (multi-head latent attention in its absorbed form).
//
// A layer of this kind projects every token to a latent c [C] and one rotated key part r [R] shared by all heads, and
// that row [c | r] (Dk = C + R values) is all the cache holds: one "KV head" per layer, no value pool. The per-head keys
// W_uk c and values W_uv c are never formed. Instead the query of head h is carried into the latent space,
// q'_h = [W_uk_h^T q_h | rotated part of q_h], so that q'_h . [c | r] is the score of the expanded key, and the context is
// gathered in the latent space too, sum_j p_j c_j [C], and expanded by W_uv_h afterwards. For the attention kernel this
// is multi-query attention whose keys have Dk dims and whose values are the first Dv = C dims of the same rows.
//
//   b200_latent_kv_store   one warp per token: RMS norm of the query latent (optional) and of c, rotary embedding of r
//                          (interleaved pairs, tables indexed by position), [c | r] -> the token's row of its cache page.
//   b200_latent_q_rope     rotated part of every query head -> columns C .. C + R of the attention's query rows.
//   b200_latent_attn       fp32 arithmetic over a 16-bit or 32-bit cache, any sizes (Dk <= 1024, Dv <= 512): a warp per
//                          (token, head), a lane per key for the scores and per column for the values.
//   b200_latent_attn_mma   bf16 on the tensor cores (mma.sync m16n8k16): the 64 rows of a CTA are (token, head) pairs of
//                          one run of consecutive tokens, all against the same key tile, so both prompt pieces (many
//                          tokens) and decode tokens (many heads) fill the M dimension. Dk % 16 == 0, Dv <= 512.
//                          `nsplit` > 1 cuts the keys of single-token tiles into ranges that are merged by a second kernel.
//
// Causal; an optional per-head sink logit enters the softmax denominator only (running maximum starts at the sink, the
// sum gains exp(sink - max) at the end).
#include "common.cuh"
#include "mma_sync.cuh"
#include "../include/b200_ops.h"

namespace b200 {

// ------------------------------------------------------------------------------------------------------------------
// latent norms + rotary + cache store
// ------------------------------------------------------------------------------------------------------------------
// proj: fp32 [tokens, ld]: columns [q_off, q_off + Cq) the query latent (Cq may be 0), [kv_off, kv_off + C) the KV latent,
// then R columns of the shared rotated key part. cq_out [tokens, Cq]; cache rows of Dk = C + R.
// One warp per token (the latents are a few hundred values: warp reductions only, no block barrier).
template <typename T, typename WT>
__global__ void __launch_bounds__(128)
latent_kv_store_kernel(const float* __restrict__ proj, long long ld, int q_off, int Cq, int kv_off, int C, int R, int rot,
                       const WT* __restrict__ wq, const WT* __restrict__ wkv, float eps, const float* __restrict__ cs,
                       const float* __restrict__ sn, const int* __restrict__ pos, const int* __restrict__ slot,
                       const int* __restrict__ table, int max_blocks, int block_size, T* __restrict__ cq_out,
                       T* __restrict__ cache, int tokens) {
  const int lane = threadIdx.x & 31;
  const long long t = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= tokens) return;
  const float* row = proj + t * ld;
  const int p = pos[t];
  const int blk = table[(long long)slot[t] * max_blocks + p / block_size];
  T* dst = cache + ((long long)blk * block_size + p % block_size) * (C + R);
  // the rotated key part first: its loads do not wait for a reduction
  const float* kr = row + kv_off + C;
  const int hr = rot / 2;
  for (int i = lane; i < hr; i += 32) {
    const float u = kr[2 * i], v = kr[2 * i + 1];
    const float c = cs[(long long)p * hr + i], s = sn[(long long)p * hr + i];
    dst[C + 2 * i] = from_f32<T>(u * c - v * s);
    dst[C + 2 * i + 1] = from_f32<T>(v * c + u * s);
  }
  for (int i = rot + lane; i < R; i += 32) dst[C + i] = from_f32<T>(kr[i]);
  float ss = 0.f, sq = 0.f;
  for (int i = lane; i < C; i += 32) { const float v = row[kv_off + i]; ss += v * v; }
  for (int i = lane; i < Cq; i += 32) { const float v = row[q_off + i]; sq += v * v; }
  ss = warp_sum(ss);
  sq = warp_sum(sq);
  const float r = 1.f / sqrtf(ss / (float)C + eps);
  for (int i = lane; i < C; i += 32) dst[i] = from_f32<T>(row[kv_off + i] * r * to_f32<WT>(wkv[i]));
  if (Cq > 0) {
    const float rq = 1.f / sqrtf(sq / (float)Cq + eps);
    for (int i = lane; i < Cq; i += 32) cq_out[t * Cq + i] = from_f32<T>(row[q_off + i] * rq * to_f32<WT>(wq[i]));
  }
}

// q [tokens, q_stride]: head h at h * (D + R), its last R columns are the rotated part -> qx[t, h, C + i]. A thread turns
// one pair; `pair2` says that pairs may be moved as one 32-bit word (16-bit type, even offsets).
template <typename T>
__global__ void __launch_bounds__(256)
latent_q_rope_kernel(const T* __restrict__ q, long long q_stride, const float* __restrict__ cs, const float* __restrict__ sn,
                     const int* __restrict__ pos, T* __restrict__ qx, int tokens, int H, int D, int R, int rot, int C, int pair2) {
  const int hr = rot / 2;
  const int items = hr + (R - rot);
  const long long per_tok = (long long)H * items;
  const long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (w >= per_tok * tokens) return;
  const long long t = w / per_tok;
  const int rem = (int)(w - t * per_tok);
  const int h = rem / items, i = rem % items;
  const int p = pos[t];
  const T* src = q + t * q_stride + (long long)h * (D + R) + D;
  T* dst = qx + (t * H + h) * (long long)(C + R) + C;
  if (i < hr) {
    float u, v;
    if (sizeof(T) == 2 && pair2) {
      const float2 f = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(src + 2 * i));
      u = f.x; v = f.y;
    } else {
      u = to_f32<T>(src[2 * i]); v = to_f32<T>(src[2 * i + 1]);
    }
    const float c = cs[(long long)p * hr + i], s = sn[(long long)p * hr + i];
    if (sizeof(T) == 2 && pair2) {
      *reinterpret_cast<uint32_t*>(dst + 2 * i) = pack_bf16x2(u * c - v * s, v * c + u * s);
    } else {
      dst[2 * i] = from_f32<T>(u * c - v * s);
      dst[2 * i + 1] = from_f32<T>(v * c + u * s);
    }
  } else {
    dst[rot + i - hr] = src[rot + i - hr];
  }
}

// ------------------------------------------------------------------------------------------------------------------
// general kernel: one warp per (token, head)
// ------------------------------------------------------------------------------------------------------------------
constexpr int kLatMaxDv = 512;
constexpr int kLatAcc = kLatMaxDv / 32;

template <typename T>
__device__ __forceinline__ float lat_dot(const float* __restrict__ q, const T* __restrict__ k, int D) {
  float acc = 0.f;
  for (int d = 0; d < D; ++d) acc = fmaf(q[d], to_f32<T>(k[d]), acc);
  return acc;
}
template <>
__device__ __forceinline__ float lat_dot<__nv_bfloat16>(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k, int D) {
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

// q [tokens, H, Dk]; cache [blocks, block_size, Dk]; out [tokens, H, Dv]
template <typename T>
__global__ void __launch_bounds__(256)
latent_attn_kernel(const T* __restrict__ q, const T* __restrict__ cache, const int* __restrict__ pos, const int* __restrict__ slot,
                   const int* __restrict__ table, int max_blocks, const float* __restrict__ sinks, T* __restrict__ out, int H,
                   int Dk, int Dv, int block_size, float scale) {
  extern __shared__ float qs[];                      // [warps, Dk]
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * (blockDim.x >> 5) + warp;
  if (h >= H) return;
  const int p = pos[t];
  const int* trow = table + (long long)slot[t] * max_blocks;
  float* myq = qs + warp * Dk;
  const T* qr = q + ((long long)t * H + h) * Dk;
  for (int d = lane; d < Dk; d += 32) myq[d] = to_f32<T>(qr[d]);
  __syncwarp();
  float m = sinks ? sinks[h] : -INFINITY;
  float l = 0.f;
  float acc[kLatAcc];
#pragma unroll
  for (int i = 0; i < kLatAcc; ++i) acc[i] = 0.f;
  for (int k0 = 0; k0 <= p; k0 += 32) {
    const int kp = k0 + lane;
    const bool valid = kp <= p;
    long long rowoff = 0;
    float sc = -INFINITY;
    if (valid) {
      rowoff = ((long long)trow[kp / block_size] * block_size + kp % block_size) * Dk;
      sc = lat_dot<T>(myq, cache + rowoff, Dk) * scale;
    }
    const float m_new = fmaxf(m, warp_max(sc));
    const float pj = valid ? expf(sc - m_new) : 0.f;
    const float resc = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * resc + warp_sum(pj);
    m = m_new;
#pragma unroll
    for (int i = 0; i < kLatAcc; ++i) acc[i] *= resc;
    const int nk = min(32, p + 1 - k0);
    for (int j = 0; j < nk; ++j) {
      const float w = __shfl_sync(0xffffffffu, pj, j);
      const long long ro = __shfl_sync(0xffffffffu, rowoff, j);
      const T* vr = cache + ro;
#pragma unroll
      for (int i = 0; i < kLatAcc; ++i) {
        const int d = lane + 32 * i;
        if (d < Dv) acc[i] = fmaf(w, to_f32<T>(vr[d]), acc[i]);
      }
    }
  }
  if (sinks) l += expf(sinks[h] - m);
  const float inv = l > 0.f ? 1.f / l : 0.f;
  T* orow = out + ((long long)t * H + h) * Dv;
#pragma unroll
  for (int i = 0; i < kLatAcc; ++i) {
    const int d = lane + 32 * i;
    if (d < Dv) orow[d] = from_f32<T>(acc[i] * inv);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// tensor-core kernel (bf16)
// ------------------------------------------------------------------------------------------------------------------
constexpr int kLQ = 64, kLK = 64;

// tiles: [n_tiles, 4] = (first row in the batch, rows <= 64, position of the first row, cache row), or NULL: tile t is the
// single token t at (pos[t], slot[t]). Grid (n_tiles * sub, head blocks, nsplit); sub = sub-tiles of 64 >> hb_log2 tokens.
// Row r of a CTA is token (r >> hb_log2) of its sub-tile and head h0 + (r & (HB - 1)).
// With NCOL = 2 the CTA has eight warps: warp w and warp w + 4 own the same 16 rows (both form the scores) and one half of
// the value columns each, which keeps the accumulators of rows of up to 512 values in registers.
// With KS (single tokens of at most 16 heads: one row group is all the CTA has) the four row-group warps all take rows 0 .. 15
// and a quarter of every key tile each, and their (max, sum, accumulator) triples are merged through shared memory at the end.
// NS key tiles are in flight or in use at a time (a decode CTA does little math per tile: what it needs is bytes in flight).
template <int DVT, int NCOL, bool KS, int NS>         // 16 * DVT * NCOL >= Dv value columns are accumulated
__global__ void __launch_bounds__(128 * NCOL)
latent_attn_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache, const int* __restrict__ tiles,
                       const int* __restrict__ pos, const int* __restrict__ slot, const int* __restrict__ table, int max_blocks,
                       const float* __restrict__ sinks, __nv_bfloat16* __restrict__ out, float* __restrict__ part, int H, int Dk,
                       int Dv, int LD, int bs_log2, int hb_log2, int sub, float scale, int nsplit) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int QR = KS ? 16 : kLQ;                    // query rows held
  __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [QR][LD]
  __nv_bfloat16* sk = sq + QR * LD;                                           // [NS][64][LD]
  const int HB = 1 << hb_log2;
  const int tq_cta = kLQ >> hb_log2;                   // tokens per CTA
  // later tiles of a piece see more keys: taking them first keeps the long CTAs out of the last wave
  const int bx = gridDim.x - 1 - blockIdx.x;
  const int tile = bx / sub, st = bx % sub;
  const int h0 = blockIdx.y * HB;
  const int split = blockIdx.z;
  int row0, nrows, pos0, srow;
  if (tiles) {
    row0 = tiles[tile * 4]; nrows = tiles[tile * 4 + 1]; pos0 = tiles[tile * 4 + 2]; srow = tiles[tile * 4 + 3];
  } else {
    row0 = tile; nrows = 1; pos0 = pos[tile]; srow = slot[tile];
  }
  const int tok0 = st * tq_cta;
  if (tok0 >= nrows) return;
  const int ntok = min(tq_cta, nrows - tok0);
  const int* trow = table + (long long)srow * max_blocks;
  const int qp0 = pos0 + tok0;                         // position of the CTA's first token
  int k_lo = 0, k_hi = qp0 + ntok;                     // keys [k_lo, k_hi)
  if (nsplit > 1) {
    const int chunk = ((k_hi + nsplit - 1) / nsplit + kLK - 1) / kLK * kLK;
    k_lo = split * chunk;
    k_hi = min(k_hi, k_lo + chunk);
  }
  const int nkb = k_hi > k_lo ? (k_hi - k_lo + kLK - 1) / kLK : 0;
  const int tid = threadIdx.x, lane = tid & 31;
  const int wq = (tid >> 5) & 3;
  const int warp = KS ? 0 : wq;                        // row group of the warp
  constexpr int NT = KS ? 2 : 8;                       // key tiles of 8 a warp scores per 64-key block, starting at tile n0
  constexpr int KK = KS ? 1 : 4;                       // k-steps of 16 keys in its P V product, starting at step kk0
  const int n0 = KS ? 2 * wq : 0, kk0 = KS ? wq : 0;
  const int col0 = (tid >> 7) * (16 * DVT);            // first value column of the warp
  const int CH = Dk >> 3, CHL = (LD - 8) >> 3;         // 16-byte chunks of a cache row / of a shared row without its pad
  const int bs_mask = (1 << bs_log2) - 1;

  // consecutive threads fetch consecutive 16-byte chunks of the tile; rows past the key range are zeroed. A thread walks its
  // chunks (row r, chunk c of the row) by increments: no division per chunk. With pages of 64 rows or more a tile lies
  // inside one page (key ranges start at multiples of 64), where its rows are back to back: chunk idx of the tile is at
  // 16 * idx bytes from the first row, so a warp's request covers 512 contiguous bytes and the page is looked up once.
  constexpr int NTHR = 128 * NCOL;
  const int ld_r0 = tid / CH, ld_c0 = tid - ld_r0 * CH, ld_dr = NTHR / CH, ld_dc = NTHR - ld_dr * CH;
  auto load_k = [&](int buf, int kb) {
    const int kp0 = k_lo + kb * kLK;
    const int nvalid = min(kLK, k_hi - kp0);
    __nv_bfloat16* dbase = sk + buf * kLK * LD;
    int r = ld_r0, c = ld_c0;
    if (bs_log2 >= 6) {
      const __nv_bfloat16* src = cache + ((((long long)trow[kp0 >> bs_log2]) << bs_log2) + (kp0 & bs_mask)) * Dk;
      for (int idx = tid; idx < kLK * CH; idx += NTHR) {
        __nv_bfloat16* dk = dbase + r * LD + c * 8;
        if (r < nvalid) cp_async16(smem_u32(dk), src + (long long)idx * 8);
        else *reinterpret_cast<uint4*>(dk) = make_uint4(0, 0, 0, 0);
        c += ld_dc; r += ld_dr;
        if (c >= CH) { c -= CH; ++r; }
      }
    } else {
      for (int idx = tid; idx < kLK * CH; idx += NTHR) {
        __nv_bfloat16* dk = dbase + r * LD + c * 8;
        const int kp = kp0 + r;
        if (r < nvalid)
          cp_async16(smem_u32(dk), cache + ((((long long)trow[kp >> bs_log2]) << bs_log2) + (kp & bs_mask)) * Dk + c * 8);
        else *reinterpret_cast<uint4*>(dk) = make_uint4(0, 0, 0, 0);
        c += ld_dc; r += ld_dr;
        if (c >= CH) { c -= CH; ++r; }
      }
    }
  };
  // columns between the row's end and the accumulated value columns (narrow rows only) stay zero in every buffer
  if (CHL > CH)
    for (int idx = tid; idx < NS * kLK * (CHL - CH); idx += NTHR)
      *reinterpret_cast<uint4*>(sk + (idx / (CHL - CH)) * LD + (CH + idx % (CHL - CH)) * 8) = make_uint4(0, 0, 0, 0);

  for (int c = tid; c < QR * CH; c += NTHR) {
    const int r = c / CH, col = (c % CH) * 8;
    const int tq = r >> hb_log2, h = h0 + (r & (HB - 1));
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tq < ntok && h < H) v = *reinterpret_cast<const uint4*>(q + ((long long)(row0 + tok0 + tq) * H + h) * Dk + col);
    *reinterpret_cast<uint4*>(sq + r * LD + col) = v;
  }
#pragma unroll
  for (int st0 = 0; st0 < NS - 1; ++st0) {               // tiles 0 .. NS - 2, a group each
    if (st0 < nkb) load_k(st0, st0);
    cp_async_commit();
  }

  const float LOG2E = 1.4426950408889634f;
  const float sl2 = scale * LOG2E;
  const int ra = warp * 16 + (lane >> 2), rb = ra + 8;
  const int ha = h0 + (ra & (HB - 1)), hb = h0 + (rb & (HB - 1));
  const int ta = ra >> hb_log2, tb = rb >> hb_log2;
  const bool va = ta < ntok && ha < H, vb = tb < ntok && hb < H;
  const bool own_sink = sinks != nullptr && nsplit == 1;
  const float sinka = own_sink && va ? sinks[ha] * LOG2E : -INFINITY;
  const float sinkb = own_sink && vb ? sinks[hb] * LOG2E : -INFINITY;
  float m0 = sinka, m1 = sinkb, l0 = 0.f, l1 = 0.f;
  float o[2 * DVT][4];
#pragma unroll
  for (int i = 0; i < 2 * DVT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const int qpa = qp0 + ta, qpb = qp0 + tb;            // positions of this thread's two rows
  // a warp none of whose rows is a token of the piece and a head of the model only helps loading
  const bool warp_live = ((warp * 16) >> hb_log2) < ntok && (HB < 16 || h0 + ((warp * 16) & (HB - 1)) < H);
  const int dkt = Dk >> 4;

  for (int kb = 0; kb < nkb; ++kb) {
    const int buf = kb % NS;
    if (kb + NS - 1 < nkb) load_k((kb + NS - 1) % NS, kb + NS - 1);
    cp_async_commit();
    cp_async_wait<NS - 1>();
    __syncthreads();
    if (warp_live) {
      const __nv_bfloat16* bk = sk + buf * kLK * LD;
      float s[NT][4];
#pragma unroll
      for (int n = 0; n < NT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
      const __nv_bfloat16* qrow = sq + (warp * 16 + (lane & 15)) * LD + (lane >> 4) * 8;
      const __nv_bfloat16* krow = bk + (n0 * 8 + (lane & 7)) * LD + (lane >> 3) * 8;
      int k = 0;
#pragma unroll 1
      for (; k + 1 < dkt; k += 2) {                      // one ldmatrix.x4 of K feeds two k-steps of a key tile
        uint32_t a[2][4], b[NT][4];
        ldsm_x4(smem_u32(qrow + k * 16), a[0][0], a[0][1], a[0][2], a[0][3]);
        ldsm_x4(smem_u32(qrow + k * 16 + 16), a[1][0], a[1][1], a[1][2], a[1][3]);
#pragma unroll
        for (int n = 0; n < NT; ++n) ldsm_x4(smem_u32(krow + n * 8 * LD + k * 16), b[n][0], b[n][1], b[n][2], b[n][3]);
#pragma unroll
        for (int n = 0; n < NT; ++n) mma_bf16_16816(s[n], a[0][0], a[0][1], a[0][2], a[0][3], b[n][0], b[n][1]);
#pragma unroll
        for (int n = 0; n < NT; ++n) mma_bf16_16816(s[n], a[1][0], a[1][1], a[1][2], a[1][3], b[n][2], b[n][3]);
      }
      if (k < dkt) {
        uint32_t a[4], b[NT][2];
        ldsm_x4(smem_u32(qrow + k * 16), a[0], a[1], a[2], a[3]);
#pragma unroll
        for (int n = 0; n < NT; ++n)
          ldsm_x2(smem_u32(bk + ((n0 + n) * 8 + (lane & 7)) * LD + k * 16 + ((lane >> 3) & 1) * 8), b[n][0], b[n][1]);
#pragma unroll
        for (int n = 0; n < NT; ++n) mma_bf16_16816(s[n], a[0], a[1], a[2], a[3], b[n][0], b[n][1]);
      }
      // causal mask and the end of the key range, only in blocks that reach past the warp's first position or the range
      const int kbase0 = k_lo + kb * kLK;
      if (kbase0 + kLK - 1 > qp0 + ((warp * 16) >> hb_log2) || kbase0 + kLK > k_hi) {
        const int kbase = kbase0 + n0 * 8 + 2 * (lane & 3);
#pragma unroll
        for (int n = 0; n < NT; ++n) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int key = kbase + n * 8 + (j & 1);
            if (key > ((j >> 1) ? qpb : qpa) || key >= k_hi) s[n][j] = -INFINITY;
          }
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
        mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0 * sl2), mn1 = fmaxf(m1, mx1 * sl2);      // scale > 0 (checked by the launcher)
      const float e0 = mn0 == -INFINITY ? 0.f : mn0, e1 = mn1 == -INFINITY ? 0.f : mn1;
      const float r0 = ex2_approx(m0 - e0), r1 = ex2_approx(m1 - e1);          // 2^(-inf) = 0 when nothing was seen yet
      m0 = mn0; m1 = mn1;
      l0 *= r0; l1 *= r1;
#pragma unroll
      for (int i = 0; i < 2 * DVT; ++i) { o[i][0] *= r0; o[i][1] *= r0; o[i][2] *= r1; o[i][3] *= r1; }
      uint32_t pa[KK][4];                                 // P as A fragments: k-steps of 16 keys
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const float p0 = ex2_approx(fmaf(s[n][0], sl2, -e0)), p1 = ex2_approx(fmaf(s[n][1], sl2, -e0));
        const float p2 = ex2_approx(fmaf(s[n][2], sl2, -e1)), p3 = ex2_approx(fmaf(s[n][3], sl2, -e1));
        l0 += p0 + p1;
        l1 += p2 + p3;
        pa[n >> 1][(n & 1) * 2] = pack_bf16x2(p0, p1);
        pa[n >> 1][(n & 1) * 2 + 1] = pack_bf16x2(p2, p3);
      }
      // the values are the first columns of the key rows
#pragma unroll
      for (int kk = 0; kk < KK; ++kk) {
#pragma unroll
        for (int n = 0; n < 2 * DVT; n += 2) {            // one ldmatrix.x4.trans feeds two output column tiles
          uint32_t b0, b1, b2, b3;
          ldsm_x4_trans(smem_u32(bk + ((kk0 + kk) * 16 + (lane & 15)) * LD + col0 + n * 8 + (lane >> 4) * 8), b0, b1, b2, b3);
          mma_bf16_16816(o[n], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
          mma_bf16_16816(o[n + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
        }
      }
    }
    __syncthreads();                                    // everyone is done with `buf` before the next prefetch lands in it
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if (KS) {
    // the four key quarters of rows 0 .. 15 meet in shared memory (the key buffers are free: the loop ended on a barrier)
    float* mg = reinterpret_cast<float*>(sk);            // [4][16][Dv + 2]
    const int W2 = Dv + 2;
    float* wa = mg + (wq * 16 + ra) * W2;
    float* wb = mg + (wq * 16 + rb) * W2;
    if ((lane & 3) == 0 && col0 == 0) {
      // the running maximum is only the reference point of the sum and the accumulators (it may be the sink's start value);
      // the sink's own term enters once, below
      wa[0] = m0; wa[1] = l0;
      wb[0] = m1; wb[1] = l1;
    }
#pragma unroll
    for (int n = 0; n < 2 * DVT; ++n) {
      const int d = col0 + n * 8 + 2 * (lane & 3);
      if (d >= Dv) continue;
      wa[2 + d] = o[n][0]; wa[3 + d] = o[n][1];
      wb[2 + d] = o[n][2]; wb[3 + d] = o[n][3];
    }
    __syncthreads();
    for (int i = tid; i < 16 * Dv; i += 128 * NCOL) {
      const int r = i / Dv, d = i - r * Dv;
      const int h = h0 + (r & (HB - 1));
      if ((r >> hb_log2) >= ntok || h >= H) continue;
      const float sk2 = own_sink ? sinks[h] * LOG2E : -INFINITY;
      float m = sk2;
#pragma unroll
      for (int w = 0; w < 4; ++w) m = fmaxf(m, mg[(w * 16 + r) * W2]);
      float l = own_sink ? exp2f(sk2 - m) : 0.f, a = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float* ws = mg + (w * 16 + r) * W2;
        if (ws[0] != -INFINITY) {
          const float e = exp2f(ws[0] - m);
          l += ws[1] * e;
          a += ws[2 + d] * e;
        }
      }
      const long long orow = (long long)(row0 + tok0 + (r >> hb_log2)) * H + h;
      if (nsplit == 1) {
        out[orow * Dv + d] = __float2bfloat16_rn(l > 0.f ? a / l : 0.f);
      } else {
        float* pr = part + (orow * nsplit + split) * W2;
        if (d == 0) { pr[0] = m; pr[1] = l; }
        pr[2 + d] = a;
      }
    }
    return;
  }
  if (nsplit == 1) {
    if (own_sink) { l0 += ex2_approx(sinka - m0); l1 += ex2_approx(sinkb - m1); }
    const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
#pragma unroll
    for (int n = 0; n < 2 * DVT; ++n) {
      const int d = col0 + n * 8 + 2 * (lane & 3);
      if (d >= Dv) continue;
      if (va)
        *reinterpret_cast<uint32_t*>(out + ((long long)(row0 + tok0 + ta) * H + ha) * Dv + d) = pack_bf16x2(o[n][0] * i0, o[n][1] * i0);
      if (vb)
        *reinterpret_cast<uint32_t*>(out + ((long long)(row0 + tok0 + tb) * H + hb) * Dv + d) = pack_bf16x2(o[n][2] * i1, o[n][3] * i1);
    }
  } else {
    // partial (max in the base-2 domain, sum, accumulators) of this key range
    float* pra = part + (((long long)(row0 + tok0 + ta) * H + ha) * nsplit + split) * (Dv + 2);
    float* prb = part + (((long long)(row0 + tok0 + tb) * H + hb) * nsplit + split) * (Dv + 2);
    if ((lane & 3) == 0 && col0 == 0) {
      if (va) { pra[0] = m0; pra[1] = l0; }
      if (vb) { prb[0] = m1; prb[1] = l1; }
    }
#pragma unroll
    for (int n = 0; n < 2 * DVT; ++n) {
      const int d = col0 + n * 8 + 2 * (lane & 3);
      if (d >= Dv) continue;
      if (va) { pra[2 + d] = o[n][0]; pra[3 + d] = o[n][1]; }
      if (vb) { prb[2 + d] = o[n][2]; prb[3 + d] = o[n][3]; }
    }
  }
}

// part [tokens, H, nsplit, Dv + 2] (maxima in the base-2 domain) -> out [tokens, H, Dv]
__global__ void latent_attn_merge_kernel(const float* __restrict__ part, const float* __restrict__ sinks,
                                         __nv_bfloat16* __restrict__ out, int H, int Dv, int nsplit) {
  const int t = blockIdx.x, h = blockIdx.y;
  const float LOG2E = 1.4426950408889634f;
  const float* pr = part + ((long long)t * H + h) * nsplit * (Dv + 2);
  const float sk = sinks ? sinks[h] * LOG2E : -INFINITY;
  float m = sk;
  for (int s = 0; s < nsplit; ++s) m = fmaxf(m, pr[s * (Dv + 2)]);
  float l = sinks ? exp2f(sk - m) : 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float ms = pr[s * (Dv + 2)];
    if (ms != -INFINITY) l += pr[s * (Dv + 2) + 1] * exp2f(ms - m);
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int d = threadIdx.x; d < Dv; d += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float ms = pr[s * (Dv + 2)];
      if (ms != -INFINITY) a += pr[s * (Dv + 2) + 2 + d] * exp2f(ms - m);
    }
    out[((long long)t * H + h) * Dv + d] = __float2bfloat16_rn(a * inv);
  }
}

template <int DVT, int NCOL, bool KS, int NS>
static int launch_latent_mma(const void* q, const void* cache, const int* tiles, int n_tiles, const int* pos, const int* slot,
                             const int* table, int max_blocks, const float* sinks, void* out, float* part, int H, int Dk, int Dv,
                             int block_size, float scale, int nsplit, cudaStream_t st) {
  const int LD = (Dk > 16 * DVT * NCOL ? Dk : 16 * DVT * NCOL) + 8;
  const size_t smem = (size_t)((KS ? 16 : kLQ) + NS * kLK) * LD * sizeof(__nv_bfloat16);
  if (smem > 227 * 1024) return B200_ERR_TOO_LARGE;
  auto kern = latent_attn_mma_kernel<DVT, NCOL, KS, NS>;
  if (smem > 48 * 1024) B200_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int bs_log2 = 0;
  while ((1 << bs_log2) < block_size) ++bs_log2;
  if ((1 << bs_log2) != block_size) return B200_ERR_UNSUPPORTED;
  // heads per CTA (a power of two): single tokens want all heads in one CTA, so that the keys are read once; pieces have
  // tokens to fill the rows with and take the split that leaves the fewest rows to padding heads (ties: more heads)
  int hb_log2 = 0;
  while ((1 << hb_log2) < H && hb_log2 < 6) ++hb_log2;
  if (tiles) {
    int best = hb_log2, waste = ((H + (1 << hb_log2) - 1) >> hb_log2 << hb_log2) - H;
    for (int c = hb_log2 - 1; c >= 0 && waste > 0; --c) {
      const int w = ((H + (1 << c) - 1) >> c << c) - H;
      if (w < waste) { best = c; waste = w; }
    }
    hb_log2 = best;
  }
  const int HB = 1 << hb_log2;
  const int sub = tiles ? HB : 1;                      // 64 tokens of a tile / (64 / HB) tokens per CTA
  dim3 grid((unsigned)n_tiles * sub, (H + HB - 1) / HB, nsplit);
  kern<<<grid, 128 * NCOL, smem, st>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, tiles, pos, slot, table, max_blocks, sinks,
                                (__nv_bfloat16*)out, part, H, Dk, Dv, LD, bs_log2, hb_log2, sub, scale, nsplit);
  B200_LAUNCH_CHECK();
  return 0;
}

}  // namespace b200

using namespace b200;

B200_API int b200_latent_kv_store(const float* proj, long long ld, int q_off, int Cq, int kv_off, int C, int R, int rot,
                                  const void* wq, const void* wkv, float eps, const float* cos_t, const float* sin_t,
                                  const int* pos, const int* slot, const int* table, int max_blocks, int block_size, void* cq_out,
                                  void* cache, int tokens, int dtype, int w_dtype, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (tokens <= 0) return 0;
  if (C <= 0 || R < 0 || rot < 0 || rot > R || (rot & 1) || Cq < 0 || block_size <= 0) return B200_ERR_BAD_SHAPE;
  typedef __nv_bfloat16 bf;
#define KS(T, WT)                                                                                                             \
  latent_kv_store_kernel<T, WT><<<(tokens + 3) / 4, 128, 0, st>>>(proj, ld, q_off, Cq, kv_off, C, R, rot, (const WT*)wq,            \
                                                                  (const WT*)wkv, eps, cos_t, sin_t, pos, slot, table, max_blocks, \
                                                                  block_size, (T*)cq_out, (T*)cache, tokens)
  if (dtype == B200_DT_BF16 && w_dtype == B200_DT_BF16) KS(bf, bf);
  else if (dtype == B200_DT_BF16 && w_dtype == B200_DT_FP32) KS(bf, float);
  else if (dtype == B200_DT_FP32 && w_dtype == B200_DT_FP32) KS(float, float);
  else if (dtype == B200_DT_FP32 && w_dtype == B200_DT_BF16) KS(float, bf);
  else return B200_ERR_UNSUPPORTED;
#undef KS
  B200_LAUNCH_CHECK();
  return 0;
}

B200_API int b200_latent_q_rope(const void* q, long long q_stride, const float* cos_t, const float* sin_t, const int* pos, void* qx,
                                int tokens, int H, int D, int R, int rot, int C, int dtype, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (tokens <= 0 || R == 0) return 0;
  if (H <= 0 || D < 0 || R < 0 || rot < 0 || rot > R || (rot & 1) || C <= 0) return B200_ERR_BAD_SHAPE;
  const long long work = (long long)tokens * H * (rot / 2 + R - rot);
  const unsigned grid = (unsigned)((work + 255) / 256);
  // a pair is one aligned 32-bit word when every offset that leads to it is even
  const int pair2 = !((q_stride | D | R | C) & 1) && !((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(qx)) & 3);
  if (dtype == B200_DT_BF16)
    latent_q_rope_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)q, q_stride, cos_t, sin_t, pos, (__nv_bfloat16*)qx,
                                                              tokens, H, D, R, rot, C, pair2);
  else if (dtype == B200_DT_FP32)
    latent_q_rope_kernel<float><<<grid, 256, 0, st>>>((const float*)q, q_stride, cos_t, sin_t, pos, (float*)qx, tokens, H, D, R, rot, C, 0);
  else return B200_ERR_UNSUPPORTED;
  B200_LAUNCH_CHECK();
  return 0;
}

B200_API int b200_latent_attn(const void* q, const void* cache, const int* pos, const int* slot, const int* table, int max_blocks,
                              const float* sinks, void* out, int tokens, int H, int Dk, int Dv, int block_size, float scale,
                              int dtype, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (tokens <= 0) return 0;
  if (H <= 0 || Dk <= 0 || Dk > 1024 || Dv <= 0 || Dv > kLatMaxDv || Dv > Dk || block_size <= 0) return B200_ERR_BAD_SHAPE;
  const int warps = H < 8 ? H : 8;
  dim3 grid(tokens, (H + warps - 1) / warps), block(32 * warps);
  const size_t smem = (size_t)warps * Dk * sizeof(float);
  if (dtype == B200_DT_BF16)
    latent_attn_kernel<__nv_bfloat16><<<grid, block, smem, st>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, pos, slot, table,
                                                                 max_blocks, sinks, (__nv_bfloat16*)out, H, Dk, Dv, block_size, scale);
  else if (dtype == B200_DT_FP32)
    latent_attn_kernel<float><<<grid, block, smem, st>>>((const float*)q, (const float*)cache, pos, slot, table, max_blocks, sinks,
                                                         (float*)out, H, Dk, Dv, block_size, scale);
  else return B200_ERR_UNSUPPORTED;
  B200_LAUNCH_CHECK();
  return 0;
}

B200_API int b200_latent_attn_mma(const void* q, const void* cache, const int* tiles, int n_tiles, const int* pos, const int* slot,
                                  const int* table, int max_blocks, const float* sinks, void* out, float* part, int H, int Dk,
                                  int Dv, int block_size, float scale, int nsplit, int dtype, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (n_tiles <= 0) return 0;
  if (dtype != B200_DT_BF16 || Dk % 16 || Dk < 16 || (Dv & 1) || Dv <= 0 || Dv > 512 || Dv > Dk || !(scale > 0.f)) return B200_ERR_UNSUPPORTED;
  if (H <= 0 || block_size <= 0 || nsplit < 1 || (nsplit > 1 && (!part || tiles)) || (!tiles && (!pos || !slot))) return B200_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(cache)) & 15) return B200_ERR_BAD_ALIGN;
  const int dvt = (Dv + 15) / 16;
  // single tokens of at most 16 heads occupy one row group: its four warps split the keys of a tile instead
  // (B200_LATENT_KEYSPLIT=0 switches that off, for measurements)
  static const bool ks_on = [] { const char* e = getenv("B200_LATENT_KEYSPLIT"); return !(e && e[0] == '0'); }();
  const bool ks = !tiles && H <= 16 && ks_on;
  // ... with three key tiles in flight where two such CTAs still fit an SM
  const int ld_max = (Dk > 16 * ((dvt + 1) / 2 * 2) ? Dk : 16 * ((dvt + 1) / 2 * 2)) + 8;
  const bool ns3 = ks && (size_t)(16 + 3 * kLK) * ld_max * sizeof(__nv_bfloat16) <= 110 * 1024;
#define LMA(N, NC, K, S) launch_latent_mma<N, NC, K, S>(q, cache, (const int*)tiles, n_tiles, pos, slot, table, max_blocks, sinks, out, \
                                                        part, H, Dk, Dv, block_size, scale, nsplit, st)
#define LM(N, NC) rc = ks ? (ns3 ? LMA(N, NC, true, 3) : LMA(N, NC, true, 2)) : LMA(N, NC, false, 2)
  int rc;
  if (dvt <= 2) LM(2, 1);
  else if (dvt <= 4) LM(4, 1);
  else if (dvt <= 6) LM(6, 1);
  else if (dvt <= 8) LM(8, 1);
  else if (dvt <= 12) LM(12, 1);
  else if (dvt <= 16) LM(16, 1);
  else if (dvt <= 24) LM(12, 2);
  else LM(16, 2);
#undef LM
#undef LMA
  if (rc) return rc;
  if (nsplit > 1) {
    latent_attn_merge_kernel<<<dim3(n_tiles, H), 64, 0, st>>>(part, sinks, (__nv_bfloat16*)out, H, Dv, nsplit);
    B200_LAUNCH_CHECK();
  }
  return 0;
}
