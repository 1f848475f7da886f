// Attention over a paged cache for a RAGGED step (rows of several sequences, a prompt's portion beside single
// decoded tokens), with the options a layer can switch on independently:
//   - per-head RMS norm of queries and keys (one weight vector of the head size, shared by the heads),
//   - rotary positions on the first `rd` dimensions, INTERLEAVED pairs (2i, 2i+1), angles from a host-made fp32
//     cos/sin table [positions, rd/2] (so any frequency scaling is the table's business),
//   - rotated values: the value of position j is turned by j over all its pairs before it is cached, and a
//     head's output at position i is turned back by -i,
//   - key/value heads shared by groups of query heads, key size D and value size V independent,
//   - a chunk mask (position i sees j <= i in its own chunk of `chunk` positions, counted from position 0) and/or
//     a sliding window (j > i - window) that may also keep the sequence's first tokens (j < first) in view,
//   - a sink: one more term exp(sink[h]) in the softmax denominator, without key or value,
//   - an output gate: head h's output times sigmoid(gate[row, h]),
//   - biases on the q / k / v projections (added here, in fp32, before norm and rotation), a layer that only makes
//     queries and reads ANOTHER layer's cached keys and values,
//   - a distance penalty: r1[h] * ln(1 + r2[h] * (i - j)) is taken off the scaled score of query i and key j.
// Scores, softmax weights and the accumulation are fp32; the cache holds E (bf16 or float).
//
// Step description as in ragged_rows.cu: row_ent[rows], ent[4 * n_ent] = (slot, first row, rows, first position);
// page_table[slot * max_pages + p] is the page of positions p*page_size .. of the sequence in that slot.
#include <math.h>

#include "mma_utils.cuh"

namespace dli {

template <typename E> __device__ __forceinline__ float a_to_f(E v);
template <> __device__ __forceinline__ float a_to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float a_to_f<bf16>(bf16 v) { return __bfloat162float(v); }
template <typename E> __device__ __forceinline__ E a_from_f(float v);
template <> __device__ __forceinline__ float a_from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 a_from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

struct AttnPrep {
  const int32_t* row_ent;
  const int32_t* ent;
  const int32_t* page_table;
  int max_pages, page_size;
  int H, G, D, V, rd;       // query heads, key/value heads, key size, value size, rotated dims of q/k
  int ldp, q_off, k_off, v_off;  // packed projection row: stride and column offsets
  const float* qn;          // [D] or NULL: weights of the query / key norm
  const float* kn;
  float eps;
  const float* cos_qk;      // [positions, rd/2] or NULL (no rotation)
  const float* sin_qk;
  const float* cos_v;       // [positions, V/2] or NULL (values are cached as they are)
  const float* sin_v;
  int table_len;
  const float* bias;        // [>= the projection's q / k / v columns] fp32 or NULL: added to the projection's columns
  int q_only;               // 1: only the queries are made; keys and values are another layer's
};

// One CTA per row; each warp takes heads in turn: q heads -> qbuf (fp32, normed and rotated), key heads and value
// heads -> the sequence's cache page.
template <typename E>
__global__ void __launch_bounds__(128)
attn_prep_append_kernel(const E* __restrict__ proj, float* __restrict__ qbuf, E* __restrict__ kc, E* __restrict__ vc,
                        AttnPrep a) {
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int4 e = reinterpret_cast<const int4*>(a.ent)[a.row_ent[row]];
  const int pos = e.w + (row - e.y);
  const int page = a.page_table[(size_t)e.x * a.max_pages + pos / a.page_size], off = pos % a.page_size;
  const E* pr = proj + (size_t)row * a.ldp;
  // grid.y spreads the heads of a row over CTAs (a decode row would otherwise walk all heads with four warps)
  const int n_items = a.q_only ? a.H : a.H + 2 * a.G;
  for (int item = blockIdx.y * 4 + warp; item < n_items; item += 4 * gridDim.y) {
    if (item < a.H + a.G) {
      const bool is_q = item < a.H;
      const int hh = is_q ? item : item - a.H;
      const int col = (is_q ? a.q_off : a.k_off) + hh * a.D;
      const E* src = pr + col;
      const float* bs = a.bias ? a.bias + col : nullptr;
      const float* nw = is_q ? a.qn : a.kn;
      float r = 1.f;
      if (nw) {
        float ss = 0.f;
        for (int c = lane; c < a.D; c += 32) { const float v = a_to_f(src[c]) + (bs ? bs[c] : 0.f); ss += v * v; }
        ss = warp_sum(ss);
        r = 1.f / sqrtf(ss / a.D + a.eps);
      }
      float* qd = qbuf + ((size_t)row * a.H + hh) * a.D;
      E* kd = kc + (((size_t)page * a.G + hh) * a.page_size + off) * a.D;
      for (int i = lane; i < a.D / 2; i += 32) {
        float u = a_to_f(src[2 * i]), v = a_to_f(src[2 * i + 1]);
        if (bs) { u += bs[2 * i]; v += bs[2 * i + 1]; }
        if (nw) { u = u * r * nw[2 * i]; v = v * r * nw[2 * i + 1]; }
        if (a.cos_qk && 2 * i < a.rd) {
          const float c = a.cos_qk[(size_t)pos * (a.rd / 2) + i], s = a.sin_qk[(size_t)pos * (a.rd / 2) + i];
          const float u2 = u * c - v * s, v2 = v * c + u * s;
          u = u2; v = v2;
        }
        if (is_q) { qd[2 * i] = u; qd[2 * i + 1] = v; }
        else { kd[2 * i] = a_from_f<E>(u); kd[2 * i + 1] = a_from_f<E>(v); }
      }
    } else {
      const int g = item - a.H - a.G;
      const E* src = pr + a.v_off + g * a.V;
      const float* bs = a.bias ? a.bias + a.v_off + g * a.V : nullptr;
      E* vd = vc + (((size_t)page * a.G + g) * a.page_size + off) * a.V;
      for (int i = lane; i < a.V / 2; i += 32) {
        float u = a_to_f(src[2 * i]), v = a_to_f(src[2 * i + 1]);
        if (bs) { u += bs[2 * i]; v += bs[2 * i + 1]; }
        if (a.cos_v) {
          const float c = a.cos_v[(size_t)pos * (a.V / 2) + i], s = a.sin_v[(size_t)pos * (a.V / 2) + i];
          const float u2 = u * c - v * s, v2 = v * c + u * s;
          u = u2; v = v2;
        }
        vd[2 * i] = a_from_f<E>(u); vd[2 * i + 1] = a_from_f<E>(v);
      }
    }
  }
}

struct AttnRun {
  const int32_t* row_ent;
  const int32_t* ent;
  const int32_t* page_table;
  int max_pages, page_size;
  int H, G, D, V;
  float scale;
  int chunk, window;        // 0 = off
  int first;                // with a chunk or window: positions below `first` stay visible whatever the lower bound says
  const float* sink;        // [H] or NULL
  int ldp, g_off;           // gate column of the packed projection row, g_off < 0: no gate
  const float* cos_v;       // [positions, V/2] or NULL: turn the output back
  const float* sin_v;
  int ldv;                  // elements between the value rows of consecutive positions (V; the key size when the
                            // values are the leading part of the key rows of one shared pool)
  int splits;               // > 1: the keys of a row are dealt to `splits` CTAs (grid.z), whose partial sums
  float* part;              // [rows, H, splits, V + 2] (unnormalised output, maximum, denominator) a merge kernel adds
  const float* r1;          // [H] or NULL: the distance penalty r1[h] * ln(1 + r2[h] * (i - j)) on the scaled scores
  const float* r2;
};

// q (shared, fp32) . k row (global): 16-byte loads where the row allows them
__device__ __forceinline__ float dot_row(const float* q, const bf16* kr, int D) {
  float d = 0.f;
  if (D % 8 == 0 && (reinterpret_cast<uintptr_t>(kr) & 15u) == 0) {
    for (int c = 0; c < D; c += 8) {
      float f[8];
      unpack8(ld_16B(kr + c), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) d = fmaf(q[c + j], f[j], d);
    }
  } else {
    for (int c = 0; c < D; ++c) d = fmaf(q[c], __bfloat162float(kr[c]), d);
  }
  return d;
}
__device__ __forceinline__ float dot_row(const float* q, const float* kr, int D) {
  float d = 0.f;
  if (D % 4 == 0 && (reinterpret_cast<uintptr_t>(kr) & 15u) == 0) {
    for (int c = 0; c < D; c += 4) {
      const float4 f = *reinterpret_cast<const float4*>(kr + c);
      d = fmaf(q[c], f.x, d); d = fmaf(q[c + 1], f.y, d); d = fmaf(q[c + 2], f.z, d); d = fmaf(q[c + 3], f.w, d);
    }
  } else {
    for (int c = 0; c < D; ++c) d = fmaf(q[c], kr[c], d);
  }
  return d;
}

// four consecutive values of a row as one load (8 bytes of bf16, 16 of float)
__device__ __forceinline__ void load4(const bf16* p, float* f) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  f[0] = bf_lo(u.x); f[1] = bf_hi(u.x); f[2] = bf_lo(u.y); f[3] = bf_hi(u.y);
}
__device__ __forceinline__ void load4(const float* p, float* f) {
  const float4 u = *reinterpret_cast<const float4*>(p);
  f[0] = u.x; f[1] = u.y; f[2] = u.z; f[3] = u.w;
}

constexpr int kAttnThreads = 128;
// The weighted value sum deals the value dimensions to threads in one of two ways.  Vector form (value size and row stride
// multiples of 4): a thread owns 4 CONSECUTIVE dimensions and reads them with one load per key; V/4 threads cover a row and
// 128 / (V/4) key groups work side by side.  Scalar form (any even V): a thread owns dimensions d0, d0 + 128, ...
__host__ __device__ inline bool attn_vec_values(int V, int ldv) { return V % 4 == 0 && ldv % 4 == 0 && kAttnThreads % (V / 4) == 0; }
__host__ __device__ inline int attn_value_groups(int V, int ldv) {
  if (attn_vec_values(V, ldv)) return kAttnThreads / (V / 4);
  return V >= kAttnThreads ? 1 : kAttnThreads / V;
}
constexpr int kAttnMaxVPerThread = 4;  // V <= 512

// One CTA per (row, query head).  Keys in tiles of 128: one score per thread, a block-wide running maximum,
// then the weighted value sum with the threads across the value dimensions (V < 128: several key groups).
template <typename E>
__global__ void __launch_bounds__(kAttnThreads)
attn_ragged_kernel(const float* __restrict__ qbuf, const E* __restrict__ kc, const E* __restrict__ vc,
                   const E* __restrict__ proj, E* __restrict__ out, AttnRun a) {
  extern __shared__ float sm[];
  float* q = sm;                      // [D]
  float* p = q + a.D;                 // [128]
  float* red = p + kAttnThreads;      // [8]
  float* ov = red + 8;                // [groups * Vpad]
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int g = h / (a.H / a.G);
  const int4 e = reinterpret_cast<const int4*>(a.ent)[a.row_ent[row]];
  const int pos = e.w + (row - e.y);
  const int32_t* pt = a.page_table + (size_t)e.x * a.max_pages;
  int lo = 0;
  if (a.chunk > 0) lo = (pos / a.chunk) * a.chunk;
  if (a.window > 0 && pos - a.window + 1 > lo) lo = pos - a.window + 1;
  for (int c = tid; c < a.D; c += kAttnThreads) q[c] = qbuf[((size_t)row * a.H + h) * a.D + c] * a.scale;
  // the visible keys are positions [0, nf) and [lo, pos]; the loops below walk them as one range of indices
  // [lo - nf, pos], an index below lo standing for position index - (lo - nf)
  const int nf = min(a.first, lo), shift = lo - nf;
  int jb = shift, je = pos;    // this CTA's keys
  if (a.splits > 1) {
    const int per = (pos - shift + a.splits) / a.splits;
    jb = shift + (int)blockIdx.z * per;
    je = min(pos, jb + per - 1);
  }
  auto key_pos = [&](int idx) { return idx < lo ? idx - shift : idx; };
  const float pen1 = a.r1 ? a.r1[h] : 0.f, pen2 = a.r1 ? a.r2[h] : 0.f;

  const bool vec = attn_vec_values(a.V, a.ldv);
  const int groups = attn_value_groups(a.V, a.ldv);
  const int my_group = vec ? tid / (a.V / 4) : (a.V >= kAttnThreads ? 0 : tid / a.V);
  const bool pv_active = my_group < groups;
  const int d0 = vec ? (tid % (a.V / 4)) * 4 : (a.V >= kAttnThreads ? tid : tid % a.V);
  const int dstep = vec ? 1 : kAttnThreads;  // acc[i] belongs to dimension d0 + i * dstep
  float acc[kAttnMaxVPerThread] = {0.f, 0.f, 0.f, 0.f};
  const bool has_sink = a.sink && blockIdx.z == 0;
  float m = has_sink ? a.sink[h] : -INFINITY;  // the sink enters as a term exp(sink - m) = 1 of the denominator
  float l = has_sink ? 1.f : 0.f;
  __syncthreads();

  for (int j0 = jb; j0 <= je; j0 += kAttnThreads) {
    // a pass of at most 64 / 32 keys (the key splits of decode rows): 2 / 4 threads share a key's dot product
    const int cnt_pass = min(kAttnThreads, je - j0 + 1);
    const int tpk = (a.D % 32 == 0) ? (cnt_pass <= 32 ? 4 : (cnt_pass <= 64 ? 2 : 1)) : 1;
    const int kidx = tid / tpk, part = tid - kidx * tpk;
    const int j = j0 + kidx;
    float s = -INFINITY;
    {
      float dpart = 0.f;
      int jp = pos;
      if (j <= je) {
        jp = key_pos(j);
        const E* kr = kc + (((size_t)pt[jp / a.page_size] * a.G + g) * a.page_size + jp % a.page_size) * a.D;
        const int len = a.D / tpk;
        dpart = dot_row(q + part * len, kr + part * len, len);
      }
      if (tpk > 1) dpart += __shfl_xor_sync(0xffffffffu, dpart, 1);
      if (tpk > 2) dpart += __shfl_xor_sync(0xffffffffu, dpart, 2);
      if (j <= je && part == 0) s = a.r1 ? dpart - pen1 * log1pf(pen2 * (float)(pos - jp)) : dpart;
    }
    // block maximum
    float mx = warp_max(s);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    const float m_new = fmaxf(m, mx);
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    const float w = (j <= je && part == 0) ? expf(s - m_new) : 0.f;
    if (part == 0) p[kidx] = w;
    float ws = warp_sum(w);
    if ((tid & 31) == 0) red[4 + (tid >> 5)] = ws;
    __syncthreads();
    l = l * corr + (red[4] + red[5] + red[6] + red[7]);
    m = m_new;
    const int cnt = min(kAttnThreads, je - j0 + 1);
#pragma unroll
    for (int i = 0; i < kAttnMaxVPerThread; ++i) acc[i] *= corr;
    if (pv_active) {
      // eight keys per round: their page lookups and value loads are all in flight before the first is used
      constexpr int KR = 8;
      for (int jj = my_group; jj < cnt; jj += KR * groups) {
        const E* vr[KR];
        float wj[KR];
#pragma unroll
        for (int u = 0; u < KR; ++u) {
          const int ju = jj + u * groups, jk = key_pos(j0 + min(ju, cnt - 1));
          vr[u] = vc + (((size_t)pt[jk / a.page_size] * a.G + g) * a.page_size + jk % a.page_size) * a.ldv;
          wj[u] = ju < cnt ? p[ju] : 0.f;
        }
        if (vec) {
          float f[KR][4];
#pragma unroll
          for (int u = 0; u < KR; ++u) load4(vr[u] + d0, f[u]);
#pragma unroll
          for (int u = 0; u < KR; ++u)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[i] = fmaf(wj[u], f[u][i], acc[i]);
        } else {
#pragma unroll
          for (int i = 0; i < kAttnMaxVPerThread; ++i) {
            const int d = d0 + i * kAttnThreads;
            if (d < a.V) {
              float f[KR];
#pragma unroll
              for (int u = 0; u < KR; ++u) f[u] = a_to_f(vr[u][d]);
#pragma unroll
              for (int u = 0; u < KR; ++u) acc[i] = fmaf(wj[u], f[u], acc[i]);
            }
          }
        }
      }
    }
  }
  // sum the key groups, normalise, turn back, gate
  __syncthreads();
  if (pv_active) {
#pragma unroll
    for (int i = 0; i < kAttnMaxVPerThread; ++i) {
      const int d = d0 + i * dstep;
      if (d < a.V) ov[my_group * a.V + d] = acc[i];
    }
  }
  __syncthreads();
  if (a.splits > 1) {
    float* pr = a.part + (((size_t)row * a.H + h) * a.splits + blockIdx.z) * (a.V + 2);
    for (int d = tid; d < a.V; d += kAttnThreads) {
      float u = 0.f;
      for (int gg = 0; gg < groups; ++gg) u += ov[gg * a.V + d];
      pr[d] = u;
    }
    if (tid == 0) { pr[a.V] = m; pr[a.V + 1] = l; }
    return;
  }
  float gate = 1.f;
  if (a.g_off >= 0) gate = 1.f / (1.f + expf(-a_to_f(proj[(size_t)row * a.ldp + a.g_off + h])));
  const float inv = 1.f / l;
  E* orow = out + ((size_t)row * a.H + h) * a.V;
  for (int i = tid; i < a.V / 2; i += kAttnThreads) {
    float u = 0.f, v = 0.f;
    for (int gg = 0; gg < groups; ++gg) { u += ov[gg * a.V + 2 * i]; v += ov[gg * a.V + 2 * i + 1]; }
    u *= inv; v *= inv;
    if (a.cos_v) {
      const float c = a.cos_v[(size_t)pos * (a.V / 2) + i], s = a.sin_v[(size_t)pos * (a.V / 2) + i];
      const float u2 = u * c + v * s, v2 = v * c - u * s;  // by -angle
      u = u2; v = v2;
    }
    orow[2 * i] = a_from_f<E>(u * gate);
    orow[2 * i + 1] = a_from_f<E>(v * gate);
  }
}

// Adds the partial sums of a row's key splits: o = sum_z e^(m_z - M) o_z / sum_z e^(m_z - M) l_z, then the same
// epilogue (turn back, gate).  One CTA per (row, head).
template <typename E>
__global__ void __launch_bounds__(kAttnThreads)
attn_ragged_merge_kernel(const E* __restrict__ proj, E* __restrict__ out, AttnRun a) {
  __shared__ float wz[64];   // e^(m_z - M) per split (0 for an empty split)
  __shared__ float lz[64];
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const float* pr = a.part + ((size_t)row * a.H + h) * a.splits * (a.V + 2);
  if (tid < 64) {
    wz[tid] = tid < a.splits ? pr[(size_t)tid * (a.V + 2) + a.V] : -INFINITY;
    lz[tid] = tid < a.splits ? pr[(size_t)tid * (a.V + 2) + a.V + 1] : 0.f;
  }
  __syncthreads();
  float M = -INFINITY;
  for (int z = 0; z < a.splits; ++z) M = fmaxf(M, wz[z]);
  __syncthreads();
  if (tid < 64) wz[tid] = wz[tid] == -INFINITY ? 0.f : expf(wz[tid] - M);
  __syncthreads();
  float L = 0.f;
  for (int z = 0; z < a.splits; ++z) L += wz[z] * lz[z];
  const int4 e = reinterpret_cast<const int4*>(a.ent)[a.row_ent[row]];
  const int pos = e.w + (row - e.y);
  float gate = 1.f;
  if (a.g_off >= 0) gate = 1.f / (1.f + expf(-a_to_f(proj[(size_t)row * a.ldp + a.g_off + h])));
  const float inv = 1.f / L;
  E* orow = out + ((size_t)row * a.H + h) * a.V;
  for (int i = tid; i < a.V / 2; i += kAttnThreads) {
    float u = 0.f, v = 0.f;
    for (int z0 = 0; z0 < a.splits; z0 += 8) {  // eight splits' loads in flight together
      float2 f[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int z = min(z0 + k, a.splits - 1);
        f[k] = *reinterpret_cast<const float2*>(pr + (size_t)z * (a.V + 2) + 2 * i);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (z0 + k < a.splits) { u = fmaf(wz[z0 + k], f[k].x, u); v = fmaf(wz[z0 + k], f[k].y, v); }
    }
    u *= inv; v *= inv;
    if (a.cos_v) {
      const float c = a.cos_v[(size_t)pos * (a.V / 2) + i], s = a.sin_v[(size_t)pos * (a.V / 2) + i];
      const float u2 = u * c + v * s, v2 = v * c - u * s;
      u = u2; v = v2;
    }
    orow[2 * i] = a_from_f<E>(u * gate);
    orow[2 * i + 1] = a_from_f<E>(v * gate);
  }
}

// ---- one key/value head shared by all query heads (latent attention over the cached rows, multi-query attention) ----
// The row-wise kernel above gives every (row, head) its own CTAs, so H heads read the same cached rows H times.  Here a CTA
// takes HPC heads of a row: a thread loads its key once and forms HPC dot products, and a value load feeds HPC accumulators.
// Plain causal mask, optional sink, key splits; values in the vector form (4 consecutive dimensions per thread).
__device__ __forceinline__ void load8(const bf16* p, float* f) { unpack8(ld_16B(p), f); }
__device__ __forceinline__ void load8(const float* p, float* f) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

template <typename E, int HPC>
__global__ void __launch_bounds__(kAttnThreads)
attn_shared_kv_kernel(const float* __restrict__ qbuf, const E* __restrict__ kc, const E* __restrict__ vc,
                      E* __restrict__ out, AttnRun a) {
  extern __shared__ float sm[];
  const int groups = attn_value_groups(a.V, a.ldv);
  float* q = sm;                               // [HPC][D]
  float* p = q + HPC * a.D;                    // [HPC][128]
  float* red = p + HPC * kAttnThreads;         // [2][HPC][4]: warp maxima, warp sums
  float* ov = red + 2 * HPC * 4;               // [groups][HPC][V]
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x, h0 = blockIdx.y * HPC, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int4 e = reinterpret_cast<const int4*>(a.ent)[a.row_ent[row]];
  const int pos = e.w + (row - e.y);
  const int32_t* pt = a.page_table + (size_t)e.x * a.max_pages;
  for (int i = tid; i < HPC * a.D; i += kAttnThreads) q[i] = qbuf[((size_t)row * a.H + h0) * a.D + i] * a.scale;
  int jb = 0, je = pos;
  if (a.splits > 1) {
    const int per = (pos + a.splits) / a.splits;
    jb = (int)blockIdx.z * per;
    je = min(pos, jb + per - 1);
  }
  const int tpg = a.V / 4;                     // threads that cover a value row
  const int my_group = tid / tpg, d0 = (tid % tpg) * 4;
  const bool pv_active = my_group < groups;
  float acc[HPC][4], m[HPC], l[HPC];
  const bool has_sink = a.sink && blockIdx.z == 0;
#pragma unroll
  for (int h = 0; h < HPC; ++h) {
    acc[h][0] = acc[h][1] = acc[h][2] = acc[h][3] = 0.f;
    m[h] = has_sink ? a.sink[h0 + h] : -INFINITY;
    l[h] = has_sink ? 1.f : 0.f;
  }
  __syncthreads();
  for (int j0 = jb; j0 <= je; j0 += kAttnThreads) {
    const int j = j0 + tid;
    const bool valid = j <= je;
    float s[HPC];
#pragma unroll
    for (int h = 0; h < HPC; ++h) s[h] = 0.f;
    if (valid) {
      const E* kr = kc + ((size_t)pt[j / a.page_size] * a.page_size + j % a.page_size) * a.D;
      int c = 0;
      for (; c + 32 <= a.D; c += 32) {  // four 16-byte key loads in flight before the first is used
        float f[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u) load8(kr + c + 8 * u, f[u]);
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int h = 0; h < HPC; ++h)
#pragma unroll
            for (int i = 0; i < 8; ++i) s[h] = fmaf(q[h * a.D + c + 8 * u + i], f[u][i], s[h]);
      }
      for (; c < a.D; c += 8) {
        float f[8];
        load8(kr + c, f);
#pragma unroll
        for (int h = 0; h < HPC; ++h)
#pragma unroll
          for (int i = 0; i < 8; ++i) s[h] = fmaf(q[h * a.D + c + i], f[i], s[h]);
      }
    }
#pragma unroll
    for (int h = 0; h < HPC; ++h) {
      if (!valid) s[h] = -INFINITY;
      const float mx = warp_max(s[h]);
      if (lane == 0) red[h * 4 + warp] = mx;
    }
    __syncthreads();
    float corr[HPC];
#pragma unroll
    for (int h = 0; h < HPC; ++h) {
      const float mx = fmaxf(fmaxf(red[h * 4], red[h * 4 + 1]), fmaxf(red[h * 4 + 2], red[h * 4 + 3]));
      const float m_new = fmaxf(m[h], mx);
      corr[h] = (m[h] == -INFINITY) ? 0.f : expf(m[h] - m_new);
      const float w = valid ? expf(s[h] - m_new) : 0.f;
      p[h * kAttnThreads + tid] = w;
      const float ws = warp_sum(w);
      if (lane == 0) red[HPC * 4 + h * 4 + warp] = ws;
      m[h] = m_new;
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < HPC; ++h) {
      const float* r2 = red + HPC * 4 + h * 4;
      l[h] = l[h] * corr[h] + (r2[0] + r2[1] + r2[2] + r2[3]);
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[h][i] *= corr[h];
    }
    const int cnt = min(kAttnThreads, je - j0 + 1);
    if (pv_active) {
      constexpr int KR = 8;  // keys per round: their page lookups and value loads are in flight together
      for (int jj = my_group; jj < cnt; jj += KR * groups) {
        float f[KR][4];
        int ju[KR];
#pragma unroll
        for (int u = 0; u < KR; ++u) {
          ju[u] = jj + u * groups;
          const int jk = j0 + min(ju[u], cnt - 1);
          load4(vc + ((size_t)pt[jk / a.page_size] * a.page_size + jk % a.page_size) * a.ldv + d0, f[u]);
        }
#pragma unroll
        for (int u = 0; u < KR; ++u) {
          if (ju[u] < cnt) {
#pragma unroll
            for (int h = 0; h < HPC; ++h) {
              const float wj = p[h * kAttnThreads + ju[u]];
#pragma unroll
              for (int i = 0; i < 4; ++i) acc[h][i] = fmaf(wj, f[u][i], acc[h][i]);
            }
          }
        }
      }
    }
    __syncthreads();  // p and red are written again by the next pass
  }
  if (pv_active) {
#pragma unroll
    for (int h = 0; h < HPC; ++h)
#pragma unroll
      for (int i = 0; i < 4; ++i) ov[((size_t)my_group * HPC + h) * a.V + d0 + i] = acc[h][i];
  }
  __syncthreads();
  for (int i = tid; i < HPC * a.V; i += kAttnThreads) {
    const int h = i / a.V, d = i - h * a.V;
    float u = 0.f;
    for (int gg = 0; gg < groups; ++gg) u += ov[((size_t)gg * HPC + h) * a.V + d];
    if (a.splits > 1) a.part[(((size_t)row * a.H + h0 + h) * a.splits + blockIdx.z) * (a.V + 2) + d] = u;
    else {
      // l of head h: every thread holds all HPC values; pick by index without dynamic register indexing
      float lh = l[0];
#pragma unroll
      for (int x = 1; x < HPC; ++x) if (h == x) lh = l[x];
      out[((size_t)row * a.H + h0 + h) * a.V + d] = a_from_f<E>(u / lh);
    }
  }
  if (a.splits > 1 && tid < HPC) {
    float mh = m[0], lh = l[0];
#pragma unroll
    for (int x = 1; x < HPC; ++x) if (tid == x) { mh = m[x]; lh = l[x]; }
    float* pr = a.part + (((size_t)row * a.H + h0 + tid) * a.splits + blockIdx.z) * (a.V + 2);
    pr[a.V] = mh;
    pr[a.V + 1] = lh;
  }
}

template <typename E, int HPC>
static int launch_shared_kv(const float* qbuf, const void* kc, const void* vc, void* out, int rows, const AttnRun& a,
                            cudaStream_t s) {
  const int groups = attn_value_groups(a.V, a.ldv);
  const size_t smem = sizeof(float) * ((size_t)HPC * a.D + HPC * kAttnThreads + 2 * HPC * 4 + (size_t)groups * HPC * a.V);
  DLI_LAUNCH("attn_shared_kv", (attn_shared_kv_kernel<E, HPC>), dim3(rows, a.H / HPC, a.splits), dim3(kAttnThreads), smem, s, qbuf,
             (const E*)kc, (const E*)vc, (E*)out, a);
  return DLI_OK;
}

// Does a step of this shape take the shared-key/value kernel, and with how many heads per CTA (0: no)?
static int shared_kv_heads(int H, int G, int D, int V, int ldv, int chunk, int window, int g_off, const float* cos_v, int dt,
                           const void* kc, const void* vc, bool has_penalty) {
  if (G != 1 || H < 2 || chunk > 0 || window > 0 || g_off >= 0 || cos_v || has_penalty) return 0;
  const size_t es = dt == 0 ? 2 : 4;
  if (D % 8 != 0 || !attn_vec_values(V, ldv) || (ldv * es) % (dt == 0 ? 8 : 16) != 0 || !aligned16(kc) ||
      (reinterpret_cast<uintptr_t>(vc) & 15u) != 0)
    return 0;
  const int hpc = H % 4 == 0 ? 4 : (H % 2 == 0 ? 2 : 0);
  if (!hpc) return 0;
  const size_t smem = sizeof(float) * ((size_t)hpc * D + hpc * kAttnThreads + 2 * hpc * 4 + (size_t)attn_value_groups(V, ldv) * hpc * V);
  return smem <= 48 * 1024 ? hpc : 0;
}

// ---- portions of prompts: the same attention on the tensor cores (bf16 caches) ---------------------------------
// One CTA per (64-row query tile of one entry, query head); 4 warps x 16 rows; key/value tiles of 64 positions
// (aligned to multiples of 64 in the sequence) staged from the pages with 16-byte cp.async, double-buffered and
// XOR-swizzled, and consumed by m16n8k16 MMAs with an fp32 online softmax, as the uniform stacks' prefill kernel
// does (attn_prefill.cu).  Differences: queries come normed and rotated from qbuf (fp32, rounded to bf16 here);
// key and value sizes are independent; the mask is per row [lo(row), row] with lo from the chunk and the window;
// the running maximum starts at the sink (in score units) with weight 1; the epilogue turns each output pair back
// by the row's position and applies the head's gate.  tiles[2t] = entry, tiles[2t+1] = first row of the tile
// within the entry.
constexpr int kRtThreads = 128;
constexpr int kRtTile = 64;

template <int DK, int DV>
__global__ void __launch_bounds__(kRtThreads)
attn_ragged_tc_kernel(const float* __restrict__ qbuf, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                      const bf16* __restrict__ proj, bf16* __restrict__ out, const int32_t* __restrict__ tiles,
                      AttnRun a) {
  constexpr int RBK = DK * 2, RBV = DV * 2, CHK = DK / 8, CHV = DV / 8;
  constexpr int kQBytes = kRtTile * RBK, kKBytes = kRtTile * RBK, kVBytes = kRtTile * RBV;
  extern __shared__ __align__(128) uint8_t smem_tc[];
  const uint32_t sQ = smem_u32(smem_tc);
  const uint32_t sK = sQ + kQBytes;
  const uint32_t sV = sK + 2 * kKBytes;
  pdl_wait();
  pdl_trigger();
  const int h = blockIdx.x, tile_id = gridDim.y - 1 - blockIdx.y;
  const int4 e = reinterpret_cast<const int4*>(a.ent)[tiles[2 * tile_id]];  // slot, row0, n, start
  const int q0 = tiles[2 * tile_id + 1];
  const int g = h / (a.H / a.G);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int32_t* pt = a.page_table + (size_t)e.x * a.max_pages;
  const int n_rows = min(kRtTile, e.z - q0);
  const int p0 = e.w + q0, p_last = p0 + n_rows - 1;

  // queries: fp32 -> bf16 into the swizzled tile
  for (int id = tid; id < kRtTile * CHK; id += kRtThreads) {
    const int row = id / CHK, c = id - row * CHK;
    uint4 u = make_uint4(0, 0, 0, 0);
    if (row < n_rows) {
      const float4* src = reinterpret_cast<const float4*>(qbuf + ((size_t)(e.y + q0 + row) * a.H + h) * DK + c * 8);
      const float4 f0 = src[0], f1 = src[1];
      u.x = pack_bf16(f0.x, f0.y); u.y = pack_bf16(f0.z, f0.w); u.z = pack_bf16(f1.x, f1.y); u.w = pack_bf16(f1.z, f1.w);
    }
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(sQ + swz<RBK>(row, c)), "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w));
  }
  // two threads per key row: one page lookup per row and tile, then that row's 16-byte pieces
  const int lrow = tid >> 1, lhalf = tid & 1;
  auto load_tile = [&](int tile, int stage) {
    const uint32_t dK = sK + stage * kKBytes, dV = sV + stage * kVBytes;
    const int tok = tile * kRtTile + lrow;
    const bool valid = tok <= p_last;
    // rows past the last position copy nothing (size 0) but still name an address: that of the last valid row, so
    // that a pool given as a window of pages is never addressed outside the window
    const int tk = valid ? tok : p_last;
    const size_t rowbase = ((size_t)pt[tk / a.page_size] * a.G + g) * a.page_size + tk % a.page_size;
    const bf16* ksrc = kc + rowbase * DK;
    const bf16* vsrc = vc + rowbase * DV;
#pragma unroll
    for (int i = 0; i < CHK / 2; ++i) {
      const int c = lhalf * (CHK / 2) + i;
      cp_async_16B(dK + swz<RBK>(lrow, c), ksrc + c * 8, valid ? 16 : 0);
    }
#pragma unroll
    for (int i = 0; i < CHV / 2; ++i) {
      const int c = lhalf * (CHV / 2) + i;
      cp_async_16B(dV + swz<RBV>(lrow, c), vsrc + c * 8, valid ? 16 : 0);
    }
  };
  auto row_lo = [&](int pos) {
    int lo = 0;
    if (a.chunk > 0) lo = (pos / a.chunk) * a.chunk;
    if (a.window > 0 && pos - a.window + 1 > lo) lo = pos - a.window + 1;
    return lo;
  };
  const int t_begin = row_lo(p0) / kRtTile, t_end = p_last / kRtTile + 1;
  // tiles of the kept first positions that lie below the first tile of the mask's range come before it
  const int t_first = min(t_begin, (min(a.first, row_lo(p0)) + kRtTile - 1) / kRtTile);
  const int n_iter = t_first + (t_end - t_begin);
  auto tile_of = [&](int it) { return it < t_first ? it : t_begin + (it - t_first); };
  const int gq = lane >> 2, t4 = lane & 3;
  const int qabs[2] = {p0 + warp * 16 + gq, p0 + warp * 16 + gq + 8};
  const int qlo[2] = {row_lo(qabs[0]), row_lo(qabs[1])};
  const float scale_log2 = a.scale * 1.4426950408889634f;
  // the sink is a score that is not scaled: in units of the raw dot product it is sink / scale
  const float m0 = a.sink ? a.sink[h] / a.scale : -INFINITY;
  // the distance penalty in the softmax's base-2 exponent: r1 ln(1 + r2 d) log2(e) = r1 log2(1 + r2 d); the scores stay
  // raw dot products, so it is taken off as pen / scale_log2
  const float pen1 = a.r1 ? a.r1[h] / scale_log2 : 0.f, pen2 = a.r1 ? a.r2[h] : 0.f;
  float m_run[2] = {m0, m0};
  float l_run[2] = {(a.sink && t4 == 0) ? 1.f : 0.f, (a.sink && t4 == 0) ? 1.f : 0.f};
  float o[DV / 8][4];
#pragma unroll
  for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  uint32_t qf[DK / 16][4];

  load_tile(tile_of(0), 0);
  cp_async_commit();
  for (int it = 0; it < n_iter; ++it) {
    const int tile = tile_of(it), stage = it & 1;
    if (it + 1 < n_iter) {
      load_tile(tile_of(it + 1), stage ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (it == 0) {
#pragma unroll
      for (int kk = 0; kk < DK / 16; ++kk) {
        const int mi = lane >> 3;
        ldmatrix_x4(qf[kk], sQ + swz<RBK>(warp * 16 + (mi & 1) * 8 + (lane & 7), kk * 2 + (mi >> 1)));
      }
    }
    const uint32_t cK = sK + stage * kKBytes, cV = sV + stage * kVBytes;
    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < DK / 16; ++kk) {
#pragma unroll
      for (int jn = 0; jn < 4; ++jn) {
        uint32_t kf[4];
        const int mi = lane >> 3;
        ldmatrix_x4(kf, cK + swz<RBK>(jn * 16 + (mi >> 1) * 8 + (lane & 7), kk * 2 + (mi & 1)));
        mma_16816(s[2 * jn], qf[kk], kf[0], kf[1]);
        mma_16816(s[2 * jn + 1], qf[kk], kf[2], kf[3]);
      }
    }
    const int tk0 = tile * kRtTile;
    if (a.r1) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const int dist = qabs[x >> 1] - (tk0 + j * 8 + 2 * t4 + (x & 1));
          s[j][x] -= pen1 * __log2f(fmaf(pen2, (float)max(dist, 0), 1.f));
        }
    }
    if (tk0 + kRtTile - 1 > p0 || tk0 < row_lo(p_last)) {  // the tile touches the diagonal or a lower bound
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const int tok = tk0 + j * 8 + 2 * t4 + (x & 1);
          const int r = x >> 1;
          if (tok > qabs[r] || (tok < qlo[r] && tok >= a.first)) s[j][x] = -INFINITY;
        }
    }
    uint32_t pa[4][4];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j) mx = fmaxf(mx, fmaxf(s[j][2 * r], s[j][2 * r + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[r], mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = (m_run[r] == -INFINITY) ? 0.f : ex2_ftz((m_run[r] - m_use) * scale_log2);
      m_run[r] = m_new;
      float rs = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float p0w = ex2_ftz((s[j][2 * r] - m_use) * scale_log2);
        const float p1w = ex2_ftz((s[j][2 * r + 1] - m_use) * scale_log2);
        rs += p0w + p1w;
        pa[j >> 1][(j & 1) * 2 + r] = pack_bf16(p0w, p1w);
      }
      l_run[r] = l_run[r] * corr + rs;
#pragma unroll
      for (int i = 0; i < DV / 8; ++i) {
        o[i][2 * r] *= corr;
        o[i][2 * r + 1] *= corr;
      }
    }
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
      for (int jp = 0; jp < DV / 16; ++jp) {
        uint32_t vf[4];
        const int mi = lane >> 3;
        ldmatrix_x4_trans(vf, cV + swz<RBV>(ks * 16 + (mi & 1) * 8 + (lane & 7), jp * 2 + (mi >> 1)));
        mma_16816(o[2 * jp], pa[ks], vf[0], vf[1]);
        mma_16816(o[2 * jp + 1], pa[ks], vf[2], vf[3]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    const int lr = warp * 16 + gq + r * 8;  // row within the tile
    if (lr < n_rows) {
      const size_t row = (size_t)e.y + q0 + lr;
      const int pos = qabs[r];
      float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
      if (a.g_off >= 0) inv *= 1.f / (1.f + expf(-__bfloat162float(proj[row * a.ldp + a.g_off + h])));
      bf16* dst = out + (row * a.H + h) * DV + 2 * t4;
#pragma unroll
      for (int i = 0; i < DV / 8; ++i) {
        float u = o[i][2 * r], v = o[i][2 * r + 1];
        if (a.cos_v) {
          const int pr = i * 4 + t4;  // pair index of columns 8i + 2*t4, +1
          const float c = a.cos_v[(size_t)pos * (DV / 2) + pr], sn = a.sin_v[(size_t)pos * (DV / 2) + pr];
          const float u2 = u * c + v * sn, v2 = v * c - u * sn;
          u = u2; v = v2;
        }
        *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(u * inv, v * inv);
      }
    }
  }
}

template <int DK, int DV>
static int launch_ragged_tc(const float* qbuf, const void* kc, const void* vc, const void* proj, void* out,
                            const int32_t* tiles, int n_tiles, const AttnRun& a, cudaStream_t s) {
  constexpr int kSmem = kRtTile * DK * 2 + 2 * kRtTile * (DK + DV) * 2;
  static PerDeviceOnce once;
  DLI_ONCE_PER_DEVICE(once, dev, DLI_CUDA_CALL(cudaFuncSetAttribute(attn_ragged_tc_kernel<DK, DV>,
                                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem)));
  DLI_LAUNCH("attn_ragged_tc", (attn_ragged_tc_kernel<DK, DV>), dim3(a.H, n_tiles), dim3(kRtThreads), (size_t)kSmem, s,
             qbuf, (const bf16*)kc, (const bf16*)vc, (const bf16*)proj, (bf16*)out, tiles, a);
  return DLI_OK;
}

}  // namespace dli

using namespace dli;

extern "C" {

int dli_attn_prep_append(const void* proj, float* qbuf, void* k_cache, void* v_cache, const int32_t* row_ent,
                         const int32_t* ent, const int32_t* page_table, int max_pages, int page_size, int rows, int H,
                         int G, int D, int V, int rd, int ldp, int q_off, int k_off, int v_off, const float* q_norm,
                         const float* k_norm, float eps, const float* cos_qk, const float* sin_qk, const float* cos_v,
                         const float* sin_v, int table_len, int dt, const float* bias, int q_only, dli_stream_t stream) {
  DLI_CHECK_ARG(proj && qbuf && (q_only || (k_cache && v_cache)) && row_ent && ent && page_table, "dli_attn_prep_append: null pointer");
  DLI_CHECK_ARG(H > 0 && G > 0 && H % G == 0 && D > 0 && V > 0 && D % 2 == 0 && V % 2 == 0 && rd % 2 == 0 && rd <= D,
                "dli_attn_prep_append: H=%d G=%d D=%d V=%d rd=%d (H %% G == 0, even sizes, rd <= D)", H, G, D, V, rd);
  DLI_CHECK_ARG((reinterpret_cast<uintptr_t>(ent) & 15u) == 0, "dli_attn_prep_append: ent must be 16-byte aligned");
  DLI_CHECK_ARG(dt == 0 || dt == 1, "element type %d: 0 = bf16, 1 = float", dt);
  if (rows <= 0) return DLI_OK;
  AttnPrep a{row_ent, ent, page_table, max_pages, page_size, H, G, D, V, rd, ldp, q_off, k_off, v_off, q_norm, k_norm,
             eps, (rd > 0 ? cos_qk : nullptr), sin_qk, cos_v, sin_v, table_len, bias, q_only ? 1 : 0};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int items = q_only ? H : H + 2 * G;
  const dim3 pgrid(rows, rows <= 64 ? (items + 3) / 4 : 1);
  if (dt == 0) DLI_LAUNCH("attn_prep_append", attn_prep_append_kernel<bf16>, pgrid, dim3(128), 0, s, (const bf16*)proj, qbuf, (bf16*)k_cache, (bf16*)v_cache, a);
  else DLI_LAUNCH("attn_prep_append", attn_prep_append_kernel<float>, pgrid, dim3(128), 0, s, (const float*)proj, qbuf, (float*)k_cache, (float*)v_cache, a);
  return DLI_OK;
}

int dli_attn_ragged(const float* qbuf, const void* k_cache, const void* v_cache, const void* proj, void* out,
                    const int32_t* row_ent, const int32_t* ent, const int32_t* page_table, int max_pages, int page_size,
                    int rows, int H, int G, int D, int V, float scale, int chunk, int window, int first, const float* sink,
                    int ldp, int g_off, const float* cos_v, const float* sin_v, int ldv, int splits, float* part, int dt,
                    const float* r1, const float* r2, dli_stream_t stream) {
  DLI_CHECK_ARG(qbuf && k_cache && v_cache && out && row_ent && ent && page_table, "dli_attn_ragged: null pointer");
  DLI_CHECK_ARG(splits >= 1 && splits <= 64 && (splits == 1 || part), "dli_attn_ragged: %d key splits (1..64, with scratch)", splits);
  DLI_CHECK_ARG(ldv == 0 || ldv >= V, "dli_attn_ragged: value row stride %d is below the value size %d", ldv, V);
  DLI_CHECK_ARG(g_off < 0 || proj, "dli_attn_ragged: a gate needs the projection rows");
  DLI_CHECK_ARG(H > 0 && G > 0 && H % G == 0 && D > 0 && V > 0 && V % 2 == 0 && V <= kAttnThreads * kAttnMaxVPerThread,
                "dli_attn_ragged: H=%d G=%d D=%d V=%d (H %% G == 0, V even and <= %d)", H, G, D, V,
                kAttnThreads * kAttnMaxVPerThread);
  DLI_CHECK_ARG(dt == 0 || dt == 1, "element type %d: 0 = bf16, 1 = float", dt);
  if (rows <= 0) return DLI_OK;
  DLI_CHECK_ARG(first >= 0, "dli_attn_ragged: %d kept first positions", first);
  DLI_CHECK_ARG((r1 == nullptr) == (r2 == nullptr), "dli_attn_ragged: the distance penalty needs both r1 and r2");
  AttnRun a{row_ent, ent, page_table, max_pages, page_size, H, G, D, V, scale, chunk, window, first, sink, ldp, g_off, cos_v,
            sin_v, ldv ? ldv : V, splits, part, r1, r2};
  const int groups = attn_value_groups(V, ldv ? ldv : V);
  const size_t smem = sizeof(float) * (D + kAttnThreads + 8 + (size_t)groups * V);
  DLI_CHECK_ARG(smem <= 48 * 1024, "dli_attn_ragged: key size %d needs %zu bytes of shared memory", D, smem);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int hpc = shared_kv_heads(H, G, D, V, ldv ? ldv : V, chunk, window, g_off, cos_v, dt, k_cache, v_cache, r1 != nullptr);
  if (hpc) {
    int rc;
    if (dt == 0) rc = hpc == 4 ? launch_shared_kv<bf16, 4>(qbuf, k_cache, v_cache, out, rows, a, s)
                               : launch_shared_kv<bf16, 2>(qbuf, k_cache, v_cache, out, rows, a, s);
    else rc = hpc == 4 ? launch_shared_kv<float, 4>(qbuf, k_cache, v_cache, out, rows, a, s)
                       : launch_shared_kv<float, 2>(qbuf, k_cache, v_cache, out, rows, a, s);
    if (rc != DLI_OK) return rc;
  } else
  if (dt == 0) DLI_LAUNCH("attn_ragged", attn_ragged_kernel<bf16>, dim3(rows, H, splits), dim3(kAttnThreads), smem, s, qbuf, (const bf16*)k_cache, (const bf16*)v_cache, (const bf16*)proj, (bf16*)out, a);
  else DLI_LAUNCH("attn_ragged", attn_ragged_kernel<float>, dim3(rows, H, splits), dim3(kAttnThreads), smem, s, qbuf, (const float*)k_cache, (const float*)v_cache, (const float*)proj, (float*)out, a);
  if (splits > 1) {
    if (dt == 0) DLI_LAUNCH("attn_ragged_merge", attn_ragged_merge_kernel<bf16>, dim3(rows, H), dim3(kAttnThreads), 0, s, (const bf16*)proj, (bf16*)out, a);
    else DLI_LAUNCH("attn_ragged_merge", attn_ragged_merge_kernel<float>, dim3(rows, H), dim3(kAttnThreads), 0, s, (const float*)proj, (float*)out, a);
  }
  return DLI_OK;
}

int dli_attn_ragged_tc_supported(int D, int V, int dt) {
  return dt == 0 && ((D == 64 && V == 64) || (D == 128 && V == 128) || (D == 64 && V == 128) || (D == 128 && V == 64) ||
                     (D == 128 && V == 256));
}

int dli_attn_ragged_tc(const float* qbuf, const void* k_cache, const void* v_cache, const void* proj, void* out,
                       const int32_t* ent, const int32_t* tiles, int n_tiles, const int32_t* page_table, int max_pages,
                       int page_size, int H, int G, int D, int V, float scale, int chunk, int window, int first,
                       const float* sink, int ldp, int g_off, const float* cos_v, const float* sin_v, const float* r1,
                       const float* r2, dli_stream_t stream) {
  DLI_CHECK_ARG(qbuf && k_cache && v_cache && out && ent && tiles && page_table, "dli_attn_ragged_tc: null pointer");
  DLI_CHECK_ARG(g_off < 0 || proj, "dli_attn_ragged_tc: a gate needs the projection rows");
  DLI_CHECK_ARG(H > 0 && G > 0 && H % G == 0 && scale > 0.f, "dli_attn_ragged_tc: H=%d G=%d scale=%g", H, G, scale);
  if (!dli_attn_ragged_tc_supported(D, V, 0))
    return dli::fail(DLI_ERR_UNSUPPORTED, "dli_attn_ragged_tc: key size %d with value size %d has no tensor-core tile", D, V);
  if (n_tiles <= 0) return DLI_OK;
  DLI_CHECK_ARG(first >= 0, "dli_attn_ragged_tc: %d kept first positions", first);
  DLI_CHECK_ARG((r1 == nullptr) == (r2 == nullptr), "dli_attn_ragged_tc: the distance penalty needs both r1 and r2");
  AttnRun a{nullptr, ent, page_table, max_pages, page_size, H, G, D, V, scale, chunk, window, first, sink, ldp, g_off, cos_v, sin_v, V, 1, nullptr, r1, r2};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (D == 64 && V == 64) return launch_ragged_tc<64, 64>(qbuf, k_cache, v_cache, proj, out, tiles, n_tiles, a, s);
  if (D == 128 && V == 128) return launch_ragged_tc<128, 128>(qbuf, k_cache, v_cache, proj, out, tiles, n_tiles, a, s);
  if (D == 64 && V == 128) return launch_ragged_tc<64, 128>(qbuf, k_cache, v_cache, proj, out, tiles, n_tiles, a, s);
  if (D == 128 && V == 64) return launch_ragged_tc<128, 64>(qbuf, k_cache, v_cache, proj, out, tiles, n_tiles, a, s);
  return launch_ragged_tc<128, 256>(qbuf, k_cache, v_cache, proj, out, tiles, n_tiles, a, s);
}

}  // extern "C"
