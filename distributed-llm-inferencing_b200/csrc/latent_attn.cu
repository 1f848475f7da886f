// Latent attention for a RAGGED step: queries and keys/values both pass through a low-rank latent, and only the
// key/value latent c [K] (RMS-normed) and one rotated key part k_r [R] shared by all heads are cached per position,
// as one row [c | k_r] of a paged pool [pages, 1, page_size, K + R].
//
// With the per-head up-projections k_h = U_k[h] c and v_h = U_v[h] c the score of head h is
//   q_n . (U_k[h] c) + q_r . k_r = (U_k[h]^T q_n) . c + q_r . k_r,
// and the head's output is U_v[h] (sum_j p_j c_j).  So attention runs over the cached rows themselves, as ONE
// key/value head shared by all query heads, with key size K + R and value = the first K entries of the key row
// (dli_attn_ragged with ldv = K + R):
//   dli_latent_prep      c_q = rmsnorm(W_dq h) -> operand of the query up-projection; c, rotated k_r -> the pool
//   dli_latent_q_absorb  q~[h] = [U_k[h]^T q_n[h] | rot(q_r[h])] -> fp32 query rows of size K + R
//   dli_latent_v_up      out[h] = (U_v[h] o~[h]) * sigmoid(gate[h])   with o~ the attention output in the latent
// Rotation: from a host-made fp32 cos/sin table [positions, R/2]; pair i is entries (2i, 2i+1) (`halves` == 0,
// interleaved) or entries (i, i + R/2) (`halves` != 0).  A model without a query latent (Q == 0) projects its
// queries directly and skips that part of dli_latent_prep.  Norms, rotation and the absorbed queries are fp32; E
// (bf16 or float) is the element type of projections and the pool.
#include <math.h>

#include "common.cuh"

namespace dli {

template <typename E> __device__ __forceinline__ float l_to_f(E v);
template <> __device__ __forceinline__ float l_to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float l_to_f<bf16>(bf16 v) { return __bfloat162float(v); }
template <typename E> __device__ __forceinline__ E l_from_f(float v);
template <> __device__ __forceinline__ float l_from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 l_from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float l_block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}

struct LatentPrep {
  const int32_t* row_ent;
  const int32_t* ent;
  const int32_t* page_table;
  int max_pages, page_size;
  int Q, K, R;              // query latent size, key/value latent size, rotated key size
  int ldp, q_off, kv_off;   // packed projection row: stride, column of the query latent, of [kv latent | k_r]
  const float* qn;          // [Q] weight of the query latent's norm
  const float* kn;          // [K] weight of the key/value latent's norm
  float eps;
  const float* cos_t;       // [positions, R/2]
  const float* sin_t;
  int halves;               // pair i of the rotated part: 0 = entries (2i, 2i+1), 1 = entries (i, i + R/2)
};

// One CTA per row.
template <typename E>
__global__ void __launch_bounds__(256)
latent_prep_kernel(const E* __restrict__ proj, E* __restrict__ cq, E* __restrict__ pool, LatentPrep a) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x, tid = threadIdx.x;
  const int4 e = reinterpret_cast<const int4*>(a.ent)[a.row_ent[row]];
  const int pos = e.w + (row - e.y);
  const size_t page = a.page_table[(size_t)e.x * a.max_pages + pos / a.page_size];
  E* dst = pool + (page * a.page_size + pos % a.page_size) * (size_t)(a.K + a.R);
  const E* pr = proj + (size_t)row * a.ldp;
  float ss = 0.f, r;
  if (a.Q > 0) {
    for (int c = tid; c < a.Q; c += blockDim.x) { const float v = l_to_f(pr[a.q_off + c]); ss += v * v; }
    ss = l_block_sum(ss, red);
    r = 1.f / sqrtf(ss / a.Q + a.eps);
    for (int c = tid; c < a.Q; c += blockDim.x) cq[(size_t)row * a.Q + c] = l_from_f<E>(l_to_f(pr[a.q_off + c]) * r * a.qn[c]);
  }
  ss = 0.f;
  for (int c = tid; c < a.K; c += blockDim.x) { const float v = l_to_f(pr[a.kv_off + c]); ss += v * v; }
  ss = l_block_sum(ss, red);
  r = 1.f / sqrtf(ss / a.K + a.eps);
  for (int c = tid; c < a.K; c += blockDim.x) dst[c] = l_from_f<E>(l_to_f(pr[a.kv_off + c]) * r * a.kn[c]);
  for (int i = tid; i < a.R / 2; i += blockDim.x) {
    const int iu = a.halves ? i : 2 * i, iv = a.halves ? i + a.R / 2 : 2 * i + 1;
    const float u = l_to_f(pr[a.kv_off + a.K + iu]), v = l_to_f(pr[a.kv_off + a.K + iv]);
    const float c = a.cos_t[(size_t)pos * (a.R / 2) + i], s = a.sin_t[(size_t)pos * (a.R / 2) + i];
    dst[a.K + iu] = l_from_f<E>(u * c - v * s);
    dst[a.K + iv] = l_from_f<E>(v * c + u * s);
  }
}

constexpr int kLatRows = 8;  // rows of a step that share one pass over a head's up-projection

// qbuf[row, h, 0:K] = sum_d q[row, h, d] * uk[h, d, :],  qbuf[row, h, K:K+R] = rot(q[row, h, D:D+R], pos); the rows of
// q are ldq elements apart (queries that are columns of a wider projection).
// Grid (row tiles, heads); threads across the K outputs, the head's D query entries of the tile's rows in shared memory.
template <typename E>
__global__ void __launch_bounds__(256)
latent_q_absorb_kernel(const E* __restrict__ q, const E* __restrict__ uk, float* __restrict__ qbuf,
                       const int32_t* __restrict__ row_ent, const int32_t* __restrict__ ent, const float* __restrict__ cos_t,
                       const float* __restrict__ sin_t, int rows, int H, int D, int R, int K, int halves, int ldq) {
  extern __shared__ float qs[];  // [kLatRows][D]
  pdl_wait();
  pdl_trigger();
  const int r0 = blockIdx.x * kLatRows, h = blockIdx.y, tid = threadIdx.x;
  const int nr = min(kLatRows, rows - r0);
  for (int i = tid; i < kLatRows * D; i += blockDim.x) {
    const int r = i / D, d = i - r * D;
    qs[i] = r < nr ? l_to_f(q[(size_t)(r0 + r) * ldq + h * (D + R) + d]) : 0.f;
  }
  __syncthreads();
  const E* w = uk + (size_t)h * D * K;
  for (int k = blockIdx.z * blockDim.x + tid; k < K; k += blockDim.x * gridDim.z) {
    if (uk == nullptr) {  // no folding: K == D, the unrotated part passes through
      for (int r = 0; r < nr; ++r) qbuf[((size_t)(r0 + r) * H + h) * (K + R) + k] = qs[r * D + k];
      continue;
    }
    float acc[kLatRows];
#pragma unroll
    for (int r = 0; r < kLatRows; ++r) acc[r] = 0.f;
    int d = 0;
    for (; d + 8 <= D; d += 8) {  // eight weight loads in flight before the first is used
      float wv[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) wv[u] = l_to_f(w[(size_t)(d + u) * K + k]);
#pragma unroll
      for (int u = 0; u < 8; ++u)
#pragma unroll
        for (int r = 0; r < kLatRows; ++r) acc[r] = fmaf(qs[r * D + d + u], wv[u], acc[r]);
    }
    for (; d < D; ++d) {
      const float wv = l_to_f(w[(size_t)d * K + k]);
#pragma unroll
      for (int r = 0; r < kLatRows; ++r) acc[r] = fmaf(qs[r * D + d], wv, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < kLatRows; ++r)
      if (r < nr) qbuf[((size_t)(r0 + r) * H + h) * (K + R) + k] = acc[r];
  }
  if (blockIdx.z != 0) return;
  for (int i = tid; i < nr * (R / 2); i += blockDim.x) {
    const int r = i / (R / 2), p = i - r * (R / 2);
    const int row = r0 + r;
    const int4 e = reinterpret_cast<const int4*>(ent)[row_ent[row]];
    const int pos = e.w + (row - e.y);
    const E* src = q + (size_t)row * ldq + h * (D + R) + D;
    const int iu = halves ? p : 2 * p, iv = halves ? p + R / 2 : 2 * p + 1;
    const float u = l_to_f(src[iu]), v = l_to_f(src[iv]);
    const float c = cos_t[(size_t)pos * (R / 2) + p], s = sin_t[(size_t)pos * (R / 2) + p];
    float* dst = qbuf + ((size_t)row * H + h) * (K + R) + K;
    dst[iu] = u * c - v * s;
    dst[iv] = v * c + u * s;
  }
}

// out[row, h*V + v] = (sum_k uv[h, v, k] * o[row, h, k]) * sigmoid(proj[row, g_off + h*V + v])   (g_off < 0: no gate)
// Grid (row tiles, heads); one warp per output v, lanes across K, the tile's latent outputs in shared memory.
template <typename E>
__global__ void __launch_bounds__(256)
latent_v_up_kernel(const E* __restrict__ o, const E* __restrict__ uv, const E* __restrict__ proj, E* __restrict__ out,
                   int rows, int H, int V, int K, int ldp, int g_off) {
  extern __shared__ float os[];  // [kLatRows][Kp], Kp = K rounded up to 256
  pdl_wait();
  pdl_trigger();
  const int r0 = blockIdx.x * kLatRows, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nr = min(kLatRows, rows - r0), nw = blockDim.x >> 5;
  const int Kp = (K + 255) / 256 * 256;
  // 16-byte weight loads give lane l entries 8l .. 8l+7 of every 256: entry j of lane l sits at j * 32 + l of its block of
  // 256, so that the lanes of a warp read consecutive words
  const bool vec = sizeof(E) == 2 && K % 8 == 0 && (reinterpret_cast<uintptr_t>(uv) & 15u) == 0;
  for (int i = tid; i < kLatRows * K; i += blockDim.x) {
    const int r = i / K, k = i - r * K;
    const int at = vec ? (k & ~255) + (k & 7) * 32 + ((k & 255) >> 3) : k;
    os[r * Kp + at] = r < nr ? l_to_f(o[((size_t)(r0 + r) * H + h) * K + k]) : 0.f;
  }
  __syncthreads();
  for (int v = blockIdx.z * nw + warp; v < V; v += nw * gridDim.z) {
    const E* w = uv + ((size_t)h * V + v) * K;
    float acc[kLatRows];
#pragma unroll
    for (int r = 0; r < kLatRows; ++r) acc[r] = 0.f;
    if (vec) {
      for (int k = lane * 8; k < K; k += 256) {  // 16 bytes of weights per lane and load
        const uint4 u4 = *reinterpret_cast<const uint4*>(w + k);
        const float w8[8] = {bf_lo(u4.x), bf_hi(u4.x), bf_lo(u4.y), bf_hi(u4.y), bf_lo(u4.z), bf_hi(u4.z), bf_lo(u4.w), bf_hi(u4.w)};
        const float* ob = os + (k & ~255) + lane;
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
          for (int r = 0; r < kLatRows; ++r) acc[r] = fmaf(ob[r * Kp + j * 32], w8[j], acc[r]);
      }
    } else {
      for (int k = lane; k < K; k += 32) {
        const float wv = l_to_f(w[k]);
#pragma unroll
        for (int r = 0; r < kLatRows; ++r) acc[r] = fmaf(os[r * Kp + k], wv, acc[r]);
      }
    }
#pragma unroll
    for (int r = 0; r < kLatRows; ++r) acc[r] = warp_sum(acc[r]);
    if (lane < nr) {
      float val = 0.f;
#pragma unroll
      for (int r = 0; r < kLatRows; ++r) if (r == lane) val = acc[r];
      const size_t row = r0 + lane;
      if (g_off >= 0) val *= 1.f / (1.f + expf(-l_to_f(proj[row * ldp + g_off + h * V + v])));
      out[(row * H + h) * V + v] = l_from_f<E>(val);
    }
  }
}

// For steps that hold portions of prompts: per-head keys [k_n | k_r] and values of every cached position of a page
// range, from kv [n, H*D + H*V] (the up-projections of the cached latents) and the pool rows [n, K + R], into pools
// of the layout the tensor-core attention reads: kx [pages, H, page_size, D + R], vx [pages, H, page_size, V].
template <typename E>
__global__ void __launch_bounds__(256)
latent_expand_kernel(const E* __restrict__ kv, const E* __restrict__ pool, E* __restrict__ kx, E* __restrict__ vx, int H,
                     int D, int R, int V, int K, int page_size) {
  pdl_wait();
  pdl_trigger();
  const size_t n = blockIdx.x;
  const size_t page = n / page_size, off = n % page_size;
  const E* kvr = kv + n * (size_t)(H * D + H * V);
  const E* pr = pool + n * (size_t)(K + R) + K;
  const int DK = D + R;
  for (int i = threadIdx.x; i < H * DK; i += blockDim.x) {
    const int h = i / DK, c = i - h * DK;
    kx[((page * H + h) * page_size + off) * DK + c] = c < D ? kvr[h * D + c] : pr[c - D];
  }
  for (int i = threadIdx.x; i < H * V; i += blockDim.x) {
    const int h = i / V, c = i - h * V;
    vx[((page * H + h) * page_size + off) * V + c] = kvr[H * D + i];
  }
}

// out[row, c] *= sigmoid(proj[row, g_off + c])
template <typename E>
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(E* __restrict__ out, const E* __restrict__ proj, int n, int ldp, int g_off) {
  pdl_wait();
  pdl_trigger();
  const size_t row = blockIdx.x;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const float g = 1.f / (1.f + expf(-l_to_f(proj[row * ldp + g_off + c])));
    out[row * n + c] = l_from_f<E>(l_to_f(out[row * n + c]) * g);
  }
}

}  // namespace dli

using namespace dli;

extern "C" {

int dli_latent_prep(const void* proj, void* cq, void* pool, const int32_t* row_ent, const int32_t* ent,
                    const int32_t* page_table, int max_pages, int page_size, int rows, int Q, int K, int R, int ldp,
                    int q_off, int kv_off, const float* q_norm, const float* kv_norm, float eps, const float* cos_t,
                    const float* sin_t, int table_len, int halves, int dt, dli_stream_t stream) {
  DLI_CHECK_ARG(proj && pool && row_ent && ent && page_table && kv_norm && (Q == 0 || (cq && q_norm)), "dli_latent_prep: null pointer");
  DLI_CHECK_ARG(Q >= 0 && K > 0 && R >= 0 && R % 2 == 0 && (R == 0 || (cos_t && sin_t && table_len > 0)),
                "dli_latent_prep: Q=%d K=%d R=%d (R even, with a rotation table)", Q, K, R);
  DLI_CHECK_ARG((reinterpret_cast<uintptr_t>(ent) & 15u) == 0, "dli_latent_prep: ent must be 16-byte aligned");
  DLI_CHECK_ARG(dt == 0 || dt == 1, "element type %d: 0 = bf16, 1 = float", dt);
  if (rows <= 0) return DLI_OK;
  LatentPrep a{row_ent, ent, page_table, max_pages, page_size, Q, K, R, ldp, q_off, kv_off, q_norm, kv_norm, eps, cos_t, sin_t, halves};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dt == 0) DLI_LAUNCH("latent_prep", latent_prep_kernel<bf16>, dim3(rows), dim3(256), 0, s, (const bf16*)proj, (bf16*)cq, (bf16*)pool, a);
  else DLI_LAUNCH("latent_prep", latent_prep_kernel<float>, dim3(rows), dim3(256), 0, s, (const float*)proj, (float*)cq, (float*)pool, a);
  return DLI_OK;
}

int dli_latent_q_absorb(const void* q, const void* uk, float* qbuf, const int32_t* row_ent, const int32_t* ent,
                        const float* cos_t, const float* sin_t, int rows, int H, int D, int R, int K, int halves, int ldq,
                        int dt, dli_stream_t stream) {
  DLI_CHECK_ARG(q && qbuf && row_ent && ent, "dli_latent_q_absorb: null pointer");
  DLI_CHECK_ARG(uk || K == D, "dli_latent_q_absorb: without an up-projection the output size is the query size");
  DLI_CHECK_ARG(H > 0 && D > 0 && K > 0 && R >= 0 && R % 2 == 0 && (R == 0 || (cos_t && sin_t)) &&
                    (size_t)kLatRows * D * sizeof(float) <= 48 * 1024,
                "dli_latent_q_absorb: H=%d D=%d R=%d K=%d", H, D, R, K);
  DLI_CHECK_ARG(dt == 0 || dt == 1, "element type %d: 0 = bf16, 1 = float", dt);
  if (rows <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // few rows (decode): a head's outputs are dealt to several CTAs of 64 threads so that the up-projection is read by many SMs
  const int th = rows <= 16 ? 64 : (K >= 256 ? 256 : 128);
  const dim3 grid((rows + kLatRows - 1) / kLatRows, H, rows <= 16 ? (K + th - 1) / th : 1);
  const size_t smem = (size_t)kLatRows * D * sizeof(float);
  if (dt == 0) DLI_LAUNCH("latent_q_absorb", latent_q_absorb_kernel<bf16>, grid, dim3(th), smem, s, (const bf16*)q, (const bf16*)uk, qbuf, row_ent, ent, cos_t, sin_t, rows, H, D, R, K, halves, ldq ? ldq : H * (D + R));
  else DLI_LAUNCH("latent_q_absorb", latent_q_absorb_kernel<float>, grid, dim3(th), smem, s, (const float*)q, (const float*)uk, qbuf, row_ent, ent, cos_t, sin_t, rows, H, D, R, K, halves, ldq ? ldq : H * (D + R));
  return DLI_OK;
}

int dli_latent_v_up(const void* o, const void* uv, const void* proj, void* out, int rows, int H, int V, int K, int ldp,
                    int g_off, int dt, dli_stream_t stream) {
  DLI_CHECK_ARG(o && uv && out && (g_off < 0 || proj), "dli_latent_v_up: null pointer");
  DLI_CHECK_ARG(H > 0 && V > 0 && K > 0 && (size_t)kLatRows * ((K + 255) / 256 * 256) * sizeof(float) <= 48 * 1024,
                "dli_latent_v_up: H=%d V=%d K=%d (K <= %d)", H, V, K, 48 * 1024 / (kLatRows * 4));
  DLI_CHECK_ARG(dt == 0 || dt == 1, "element type %d: 0 = bf16, 1 = float", dt);
  if (rows <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid((rows + kLatRows - 1) / kLatRows, H, rows <= 16 ? (V + 31) / 32 : 1);
  const size_t smem = (size_t)kLatRows * ((K + 255) / 256 * 256) * sizeof(float);
  if (dt == 0) DLI_LAUNCH("latent_v_up", latent_v_up_kernel<bf16>, grid, dim3(256), smem, s, (const bf16*)o, (const bf16*)uv, (const bf16*)proj, (bf16*)out, rows, H, V, K, ldp, g_off);
  else DLI_LAUNCH("latent_v_up", latent_v_up_kernel<float>, grid, dim3(256), smem, s, (const float*)o, (const float*)uv, (const float*)proj, (float*)out, rows, H, V, K, ldp, g_off);
  return DLI_OK;
}

int dli_latent_expand(const void* kv, const void* pool, void* kx, void* vx, int n, int H, int D, int R, int V, int K,
                      int page_size, int dt, dli_stream_t stream) {
  DLI_CHECK_ARG(kv && pool && kx && vx && H > 0 && D > 0 && V > 0 && K > 0 && R >= 0 && page_size > 0 && n % page_size == 0,
                "dli_latent_expand: null pointer or bad shape");
  DLI_CHECK_ARG(dt == 0 || dt == 1, "element type %d: 0 = bf16, 1 = float", dt);
  if (n <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dt == 0) DLI_LAUNCH("latent_expand", latent_expand_kernel<bf16>, dim3(n), dim3(256), 0, s, (const bf16*)kv, (const bf16*)pool, (bf16*)kx, (bf16*)vx, H, D, R, V, K, page_size);
  else DLI_LAUNCH("latent_expand", latent_expand_kernel<float>, dim3(n), dim3(256), 0, s, (const float*)kv, (const float*)pool, (float*)kx, (float*)vx, H, D, R, V, K, page_size);
  return DLI_OK;
}

int dli_sigmoid_gate(void* out, const void* proj, int rows, int n, int ldp, int g_off, int dt, dli_stream_t stream) {
  DLI_CHECK_ARG(out && proj && n > 0 && g_off >= 0 && ldp >= g_off + n, "dli_sigmoid_gate: null pointer or bad shape");
  DLI_CHECK_ARG(dt == 0 || dt == 1, "element type %d: 0 = bf16, 1 = float", dt);
  if (rows <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dt == 0) DLI_LAUNCH("sigmoid_gate", sigmoid_gate_kernel<bf16>, dim3(rows), dim3(256), 0, s, (bf16*)out, (const bf16*)proj, n, ldp, g_off);
  else DLI_LAUNCH("sigmoid_gate", sigmoid_gate_kernel<float>, dim3(rows), dim3(256), 0, s, (float*)out, (const float*)proj, n, ldp, g_off);
  return DLI_OK;
}

}  // extern "C"
