// Row-wise pieces of a model whose residual stream is fp32 and whose batch is RAGGED: the rows of one step are
// portions of different sequences (a prompt's next tokens beside single decoded tokens).  A step is described
// by two int32 arrays: row_ent[rows] (which entry a row belongs to) and ent[4 * n_ent] = (state slot, first row,
// number of rows, position of the first row) per entry.
//
//   embedding -> fp32 rows, one-number RMS norm, post-norm residual add fused with the next pre-norm,
//   causal per-channel convolution over time with a per-slot tail state, row gather, a plain tiled GEMM
//   for element types / shapes the tensor-core GEMM does not take, silu(gate) * up.
//
// Element type E of weights and activations: bf16 (dt = 0) or float (dt = 1).  Norms, the convolution and the
// residual are fp32 for both.
#include "common.cuh"

namespace dli {

template <typename E> __device__ __forceinline__ float to_f(E v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }
template <typename E> __device__ __forceinline__ E from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();  // red may still be read from a previous call
  if ((threadIdx.x & 31) == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}

// x[row] = table[ids[row]] * scale as fp32 (the residual stream starts in fp32).  With inv_freq [ceil(d/2)] a sinusoidal
// position vector is added: channel 2i gets sin(p * inv_freq[i]), channel 2i+1 the cosine, p the row's position in its
// sequence (from row_ent / ent), angle and functions in fp32.
template <typename E>
__global__ void __launch_bounds__(1024)
embedding_f32_kernel(const int32_t* __restrict__ ids, const E* __restrict__ table, float* __restrict__ x,
                     float* __restrict__ x2, E* __restrict__ xe, int d, int vocab, float scale,
                     const int32_t* __restrict__ row_ent, const int32_t* __restrict__ ent,
                     const float* __restrict__ inv_freq) {
  pdl_wait();
  pdl_trigger();
  const size_t row = blockIdx.x;
  int id = ids[row];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  float pos = 0.f;
  if (inv_freq) {
    const int4 e = reinterpret_cast<const int4*>(ent)[row_ent[row]];
    pos = (float)(e.w + ((int)row - e.y));
  }
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float v = to_f(table[(size_t)id * d + c]) * scale;
    if (inv_freq) {
      const float ang = pos * inv_freq[c >> 1];
      v += (c & 1) ? cosf(ang) : sinf(ang);
    }
    x[row * d + c] = v;
    if (x2) x2[row * d + c] = v;
    if (xe) xe[row * d + c] = from_f<E>(v);
  }
}

// RMS norm in GROUPS with a weight per channel: the row is cut into `groups` equal consecutive parts, each divided
// by its own sqrt(mean(part^2) + eps), the whole multiplied by w.  hn (fp32) and he (element type E) are both
// optional outputs: a layer whose mixer reads the normed row through an fp32 convolution while its feed-forward
// reads it as a GEMM operand wants both.
template <typename E>
__global__ void __launch_bounds__(1024)
group_rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ hn,
                     E* __restrict__ he, int d, int groups, float eps) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const size_t o = (size_t)blockIdx.x * d;
  const int gd = d / groups;
  for (int g = 0; g < groups; ++g) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < gd; c += blockDim.x) { const float v = x[o + g * gd + c]; ss += v * v; }
    ss = block_sum(ss, red);
    const float r = 1.f / sqrtf(ss / gd + eps);
    for (int c = threadIdx.x; c < gd; c += blockDim.x) {
      const float v = x[o + g * gd + c] * r * w[g * gd + c];
      if (hn) hn[o + g * gd + c] = v;
      if (he) he[o + g * gd + c] = from_f<E>(v);
    }
  }
}

// Decode rows (one row per entry): the grouped norm AND the mixer's input convolution with its tail shift in one
// kernel: hn / he as above, hc = h + conv(h) in the element type (the row's CTA is the only reader and writer of its
// slot's tail).
constexpr int kMaxNormGroups = 64;
template <typename E>
__global__ void __launch_bounds__(1024)
group_rmsnorm_conv_single_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ hn,
                                 E* __restrict__ he, float* __restrict__ tail, const float* __restrict__ cw,
                                 const int32_t* __restrict__ ent, E* __restrict__ hc, int d, int groups, float eps, int taps) {
  __shared__ float red[32];
  __shared__ float rg[kMaxNormGroups];
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x;
  const size_t o = (size_t)row * d;
  const int gd = d / groups;
  for (int g = 0; g < groups; ++g) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < gd; c += blockDim.x) { const float v = x[o + g * gd + c]; ss += v * v; }
    ss = block_sum(ss, red);
    if (threadIdx.x == 0) rg[g] = 1.f / sqrtf(ss / gd + eps);
  }
  __syncthreads();
  const int4 e = reinterpret_cast<const int4*>(ent)[row];  // slot, row0 (== row), 1, position
  const int keep = taps - 1;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float cur = x[o + c] * rg[c / gd] * w[c];
    if (hn) hn[o + c] = cur;
    if (he) he[o + c] = from_f<E>(cur);
    float* t = tail + (size_t)e.x * keep * d + c;
    float acc = cw[(size_t)c * taps + keep] * cur;
    for (int i = 0; i < keep; ++i) {  // tail slot i holds position pos - keep + i
      const float v = (e.w - keep + i >= 0) ? t[(size_t)i * d] : 0.f;
      acc += cw[(size_t)c * taps + i] * v;
      if (i > 0) t[(size_t)(i - 1) * d] = v;
    }
    if (keep > 0) t[(size_t)(keep - 1) * d] = cur;
    hc[o + c] = from_f<E>(cur + acc);
  }
}

// x += y1 + y2 + a[row] * h: the residual add of a layer whose sublayers run side by side on one normed input
// (y2, and a with h, optional; a[row] is the weight of the branches that pass their input through unchanged).
template <typename E>
__global__ void __launch_bounds__(256)
residual_add2_kernel(float* __restrict__ x, const E* __restrict__ y1, const E* __restrict__ y2,
                     const float* __restrict__ a, const float* __restrict__ h, int d) {
  pdl_wait();
  pdl_trigger();
  const size_t o = (size_t)blockIdx.x * d;
  const float aw = a ? a[blockIdx.x] : 0.f;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < d; c += blockDim.x * gridDim.y) {
    float v = to_f(y1[o + c]);
    if (y2) v += to_f(y2[o + c]);
    if (a) v += aw * h[o + c];
    x[o + c] += v;
  }
}

// out[row] = E([a[row] | b[row]]): two fp32 rows side by side as one GEMM operand.
template <typename E>
__global__ void __launch_bounds__(256)
concat_cast_kernel(const float* __restrict__ a, const float* __restrict__ b, E* __restrict__ out, int d) {
  pdl_wait();
  pdl_trigger();
  const size_t r = blockIdx.x;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    out[r * 2 * d + c] = from_f<E>(a[r * d + c]);
    out[r * 2 * d + d + c] = from_f<E>(b[r * d + c]);
  }
}

// x[row] = y[row] + bias: a projection's output becomes the fp32 residual stream.
template <typename E>
__global__ void __launch_bounds__(256)
rows_bias_f32_kernel(const E* __restrict__ y, const float* __restrict__ bias, float* __restrict__ x, int d) {
  pdl_wait();
  pdl_trigger();
  const size_t o = (size_t)blockIdx.x * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) x[o + c] = to_f(y[o + c]) + (bias ? bias[c] : 0.f);
}

// hn = x / sqrt(mean(x^2) + eps) * g  with ONE weight g for the whole row.
__global__ void __launch_bounds__(1024)
scalar_rmsnorm_kernel(const float* __restrict__ x, float* __restrict__ hn, int d, float eps, float g) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const float* xr = x + (size_t)blockIdx.x * d;
  float ss = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) ss += xr[c] * xr[c];
  ss = block_sum(ss, red);
  const float r = g / sqrtf(ss / d + eps);
  for (int c = threadIdx.x; c < d; c += blockDim.x) hn[(size_t)blockIdx.x * d + c] = xr[c] * r;
}

// x += y / sqrt(mean(y^2) + eps) * g_post; then (hn != NULL) hn = x / sqrt(mean(x^2) + eps) * g_next:
// the post-norm of one sublayer, the fp32 residual add and the pre-norm of the next sublayer in one pass.
template <typename E>
__global__ void __launch_bounds__(1024)
postnorm_add_norm_kernel(const E* __restrict__ y, float* __restrict__ x, float* __restrict__ hn, int d, float eps,
                         float g_post, float g_next) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const size_t o = (size_t)blockIdx.x * d;
  float ss = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float v = to_f(y[o + c]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float r = g_post / sqrtf(ss / d + eps);
  float s2 = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float v = x[o + c] + to_f(y[o + c]) * r;
    x[o + c] = v;
    s2 += v * v;
  }
  if (hn == nullptr) return;
  s2 = block_sum(s2, red);
  const float r2 = g_next / sqrtf(s2 / d + eps);
  for (int c = threadIdx.x; c < d; c += blockDim.x) hn[o + c] = x[o + c] * r2;
}

// out[t] = h[t] + sum_j w[:, j] * h[t - taps + 1 + j]: a causal convolution over time on each channel.  Rows
// before the entry's first row come from `tail` [slots, taps - 1, d] (the last taps - 1 inputs of the sequence,
// oldest first); positions before the sequence's start are zero whatever the slot held before.
template <typename E>
__global__ void __launch_bounds__(256)
causal_conv_kernel(const float* __restrict__ h, const float* __restrict__ tail, const float* __restrict__ w,
                   const int32_t* __restrict__ row_ent, const int32_t* __restrict__ ent, E* __restrict__ out, int d,
                   int taps) {
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x;
  const int4 e = reinterpret_cast<const int4*>(ent)[row_ent[row]];  // slot, row0, n, start
  const int back = row - e.y, pos = e.w + back;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int dist = taps - 1 - j;
      if (pos - dist < 0) continue;
      float v;
      if (dist <= back) v = h[(size_t)(row - dist) * d + c];
      else v = tail[((size_t)e.x * (taps - 1) + (taps - 1 - (dist - back))) * d + c];
      acc += w[(size_t)c * taps + j] * v;
    }
    out[(size_t)row * d + c] = from_f<E>(h[(size_t)row * d + c] + acc);
  }
}

// The same for a step in which every entry brings ONE row (decode): the row's CTA is the only reader and writer of
// its slot's tail, so the convolution and the tail's shift are one kernel.
template <typename E>
__global__ void __launch_bounds__(256)
causal_conv_single_kernel(const float* __restrict__ h, float* __restrict__ tail, const float* __restrict__ w,
                          const int32_t* __restrict__ ent, E* __restrict__ out, int d, int taps) {
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x;
  const int4 e = reinterpret_cast<const int4*>(ent)[row];  // slot, row0 (== row), 1, position
  const int keep = taps - 1;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float* t = tail + (size_t)e.x * keep * d + c;
    const float cur = h[(size_t)row * d + c];
    float acc = w[(size_t)c * taps + keep] * cur;
    for (int i = 0; i < keep; ++i) {  // tail slot i holds position pos - keep + i
      const float v = (e.w - keep + i >= 0) ? t[(size_t)i * d] : 0.f;
      acc += w[(size_t)c * taps + i] * v;
      if (i > 0) t[(size_t)(i - 1) * d] = v;
    }
    if (keep > 0) t[(size_t)(keep - 1) * d] = cur;
    out[(size_t)row * d + c] = from_f<E>(cur + acc);
  }
}

// Decode rows (one row per entry): the post-norm of a sublayer, the fp32 residual add, the pre-norm of the next
// sublayer AND that sublayer's input convolution with its tail shift in one kernel (y == NULL: no post-norm part,
// the row of x is normed and convolved as it is — the first sublayer after the embedding).
template <typename E>
__global__ void __launch_bounds__(1024)
postnorm_add_norm_conv_single_kernel(const E* __restrict__ y, float* __restrict__ x, float* __restrict__ tail,
                                     const float* __restrict__ w, const int32_t* __restrict__ ent, E* __restrict__ out,
                                     int d, int taps, float eps, float g_post, float g_next) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x;
  const size_t o = (size_t)row * d;
  float s2 = 0.f;
  if (y != nullptr) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
      const float v = to_f(y[o + c]);
      ss += v * v;
    }
    ss = block_sum(ss, red);
    const float r = g_post / sqrtf(ss / d + eps);
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
      const float v = x[o + c] + to_f(y[o + c]) * r;
      x[o + c] = v;
      s2 += v * v;
    }
  } else {
    for (int c = threadIdx.x; c < d; c += blockDim.x) s2 += x[o + c] * x[o + c];
  }
  s2 = block_sum(s2, red);
  const float r2 = g_next / sqrtf(s2 / d + eps);
  const int4 e = reinterpret_cast<const int4*>(ent)[row];
  const int keep = taps - 1;
  constexpr int kMaxKeep = 7;  // up to 8 taps: all tail values and weights of a channel are loaded before any is used
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float* t = tail + (size_t)e.x * keep * d + c;
    const float cur = x[o + c] * r2;
    if (keep <= kMaxKeep) {
      float tv[kMaxKeep], wv[kMaxKeep + 1];
#pragma unroll
      for (int i = 0; i < kMaxKeep; ++i) {
        tv[i] = (i < keep && e.w - keep + i >= 0) ? t[(size_t)i * d] : 0.f;
        wv[i] = i < keep ? w[(size_t)c * taps + i] : 0.f;
      }
      float acc = w[(size_t)c * taps + keep] * cur;
#pragma unroll
      for (int i = 0; i < kMaxKeep; ++i) {
        if (i < keep) {
          acc += wv[i] * tv[i];
          if (i > 0) t[(size_t)(i - 1) * d] = tv[i];
        }
      }
      if (keep > 0) t[(size_t)(keep - 1) * d] = cur;
      out[o + c] = from_f<E>(cur + acc);
      continue;
    }
    float acc = w[(size_t)c * taps + keep] * cur;
    for (int i = 0; i < keep; ++i) {
      const float v = (e.w - keep + i >= 0) ? t[(size_t)i * d] : 0.f;
      acc += w[(size_t)c * taps + i] * v;
      if (i > 0) t[(size_t)(i - 1) * d] = v;
    }
    t[(size_t)(keep - 1) * d] = cur;
    out[o + c] = from_f<E>(cur + acc);
  }
}

// After the convolution of a step: the tail of every entry's slot becomes the last taps - 1 inputs of the sequence.
__global__ void __launch_bounds__(256)
conv_tail_update_kernel(const float* __restrict__ h, float* __restrict__ tail, const int32_t* __restrict__ ent, int d,
                        int taps) {
  pdl_wait();
  pdl_trigger();
  const int4 e = reinterpret_cast<const int4*>(ent)[blockIdx.x];
  const int keep = taps - 1, end = e.w + e.z;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float* t = tail + (size_t)e.x * keep * d + c;
    for (int i = 0; i < keep; ++i) {  // ascending: slot i reads old slot i + n (n >= 1), never one already written
      const int p = end - keep + i;
      float v = 0.f;
      if (p >= e.w) v = h[(size_t)(e.y + p - e.w) * d + c];
      else if (p >= 0) v = t[(size_t)(keep - (e.w - p)) * d];
      t[(size_t)i * d] = v;
    }
  }
}

// out[i] = E(src[rows[i]])
template <typename E>
__global__ void __launch_bounds__(256)
gather_cast_kernel(const float* __restrict__ src, const int32_t* __restrict__ rows, E* __restrict__ out, int d) {
  pdl_wait();
  pdl_trigger();
  const size_t r = rows[blockIdx.x];
  for (int c = threadIdx.x; c < d; c += blockDim.x) out[(size_t)blockIdx.x * d + c] = from_f<E>(src[r * d + c]);
}

// y[M,N] = x[M,K] . w[N,K]^T, fp32 accumulation on the CUDA cores (true fp32 for float operands).  64x64 tile,
// 16 deep, 4x4 outputs per thread.  Any M, N, K; rows of x and y may be strided.
template <typename E, typename O>
__global__ void __launch_bounds__(256)
linear_any_kernel(const E* __restrict__ x, const E* __restrict__ w, O* __restrict__ y, int M, int N, int K, int ldx,
                  int ldy) {
  __shared__ float xs[16][64 + 4];
  __shared__ float ws[16][64 + 4];
  pdl_wait();
  pdl_trigger();
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
      const int r = i >> 4, k = i & 15;
      xs[k][r] = (m0 + r < M && k0 + k < K) ? to_f(x[(size_t)(m0 + r) * ldx + k0 + k]) : 0.f;
      ws[k][r] = (n0 + r < N && k0 + k < K) ? to_f(w[(size_t)(n0 + r) * K + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < M && n < N) y[(size_t)m * ldy + n] = from_f<O>(acc[i][j]);
    }
}

// act[m, f] = silu(gu[m, f] + b[f]) * (gu[m, F + f] + b[F + f]); bias [2F] fp32 or NULL
template <typename E>
__global__ void __launch_bounds__(256)
silu_mul_kernel(const E* __restrict__ gu, E* __restrict__ act, int F, int ld, const float* __restrict__ bias, int vec) {
  pdl_wait();
  pdl_trigger();
  const size_t m = blockIdx.x;
  if (vec) {
    // 16 bytes per access: V consecutive channels of the gate half and of the up half
    constexpr int V = 16 / (int)sizeof(E);
    for (int f = (blockIdx.y * blockDim.x + threadIdx.x) * V; f < F; f += blockDim.x * gridDim.y * V) {
      float g[V], u[V], o[V];
      if constexpr (sizeof(E) == 2) {
        unpack8(ld_16B(gu + m * ld + f), g);
        unpack8(ld_16B(gu + m * ld + F + f), u);
      } else {
        const float4 a4 = *reinterpret_cast<const float4*>(gu + m * ld + f), b4 = *reinterpret_cast<const float4*>(gu + m * ld + F + f);
        g[0] = a4.x; g[1] = a4.y; g[2] = a4.z; g[3] = a4.w;
        u[0] = b4.x; u[1] = b4.y; u[2] = b4.z; u[3] = b4.w;
      }
#pragma unroll
      for (int k = 0; k < V; ++k) {
        if (bias) { g[k] += bias[f + k]; u[k] += bias[F + f + k]; }
        o[k] = to_f(from_f<E>(silu_f(g[k]))) * u[k];
      }
      if constexpr (sizeof(E) == 2) st_16B(act + m * F + f, pack8(o));
      else *reinterpret_cast<float4*>(act + m * F + f) = make_float4(o[0], o[1], o[2], o[3]);
    }
    return;
  }
  for (int f = blockIdx.y * blockDim.x + threadIdx.x; f < F; f += blockDim.x * gridDim.y) {
    float g = to_f(gu[m * ld + f]), u = to_f(gu[m * ld + F + f]);
    if (bias) { g += bias[f]; u += bias[F + f]; }
    act[m * F + f] = from_f<E>(to_f(from_f<E>(silu_f(g))) * u);
  }
}


// x += y / sqrt(mean(y^2) + eps) * w with a weight PER CHANNEL (y == NULL: x stays), then he = E(x) when he is given:
// the post-norm of a sublayer whose successor reads the residual stream itself, as a GEMM operand.
template <typename E>
__global__ void __launch_bounds__(1024)
postnorm_vec_add_kernel(const E* __restrict__ y, float* __restrict__ x, const float* __restrict__ w, E* __restrict__ he,
                        int d, float eps) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const size_t o = (size_t)blockIdx.x * d;
  float r = 0.f;
  if (y) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) { const float v = to_f(y[o + c]); ss += v * v; }
    ss = block_sum(ss, red);
    r = 1.f / sqrtf(ss / d + eps);
  }
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float v = x[o + c];
    if (y) { v += to_f(y[o + c]) * r * w[c]; x[o + c] = v; }
    if (he) he[o + c] = from_f<E>(v);
  }
}

// Per-layer token input, first half: g[row, c] = gelu_tanh(s[row, c]) * table[ids[row], off + c].
template <typename E>
__global__ void __launch_bounds__(256)
token_side_act_kernel(const E* __restrict__ s, const int32_t* __restrict__ ids, const E* __restrict__ table,
                      E* __restrict__ g, int n, int ld_tab, int off, int vocab) {
  pdl_wait();
  pdl_trigger();
  const size_t row = blockIdx.x;
  int id = ids[row];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  for (int c = threadIdx.x; c < n; c += blockDim.x)
    g[row * n + c] = from_f<E>(gelu_new_f(to_f(s[row * n + c])) * to_f(table[(size_t)id * ld_tab + off + c]));
}

// The whole per-layer token input for few rows (decode): y = Wp (gelu_tanh(Wg x) * table[id, off : off + n]),
// x += y / sqrt(mean(y^2) + eps) * w, he = E(x).  One CTA per row; the row, the n gate values and y stay in shared
// memory, products and sums are fp32.
template <typename E>
__global__ void __launch_bounds__(1024)
token_side_kernel(float* __restrict__ x, const int32_t* __restrict__ ids, const E* __restrict__ table,
                  const E* __restrict__ wg, const E* __restrict__ wp, const float* __restrict__ w, E* __restrict__ he,
                  int d, int n, int ld_tab, int off, int vocab, float eps) {
  extern __shared__ float sm_side[];
  float* xs = sm_side;       // [d]
  float* ys = xs + d;        // [d]
  float* gs = ys + d;        // [n]
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const size_t o = (size_t)blockIdx.x * d;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  int id = ids[blockIdx.x];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  for (int c = threadIdx.x; c < d; c += blockDim.x) xs[c] = x[o + c];
  __syncthreads();
  for (int c = warp; c < n; c += nw) {
    const E* wr = wg + (size_t)c * d;
    float acc = 0.f;
    for (int k = lane; k < d; k += 32) acc = fmaf(to_f(wr[k]), xs[k], acc);
    acc = warp_sum(acc);
    if (lane == 0) gs[c] = gelu_new_f(acc) * to_f(table[(size_t)id * ld_tab + off + c]);
  }
  __syncthreads();
  float ss = 0.f;
  for (int k = threadIdx.x; k < d; k += blockDim.x) {
    const E* wr = wp + (size_t)k * n;
    float acc = 0.f;
    for (int c = 0; c < n; ++c) acc = fmaf(to_f(wr[c]), gs[c], acc);
    ys[k] = acc;
    ss = fmaf(acc, acc, ss);
  }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / d + eps);
  for (int k = threadIdx.x; k < d; k += blockDim.x) {
    const float v = xs[k] + ys[k] * r * w[k];
    x[o + k] = v;
    if (he) he[o + k] = from_f<E>(v);
  }
}

// Per-layer token input for few rows, first half as ONE kernel: g[row, c] = gelu_tanh(w_gate[c] . x[row]) *
// table[ids[row], off + c], read from the fp32 residual row itself.  Grid (rows, ceil(n / 8)): a warp per gate channel.
template <typename E>
__global__ void __launch_bounds__(256)
token_side_gate_kernel(const float* __restrict__ x, const int32_t* __restrict__ ids, const E* __restrict__ table,
                       const E* __restrict__ wg, E* __restrict__ g, int d, int n, int ld_tab, int off, int vocab) {
  pdl_wait();
  pdl_trigger();
  const size_t row = blockIdx.x;
  const int lane = threadIdx.x & 31, c = blockIdx.y * 8 + (threadIdx.x >> 5);
  if (c >= n) return;
  const float* xr = x + row * d;
  const E* wr = wg + (size_t)c * d;
  float acc = 0.f;
  if (sizeof(E) == 2 && d % 8 == 0 && (reinterpret_cast<uintptr_t>(wr) & 15u) == 0) {
    // 16 bytes of weights (8 entries) per lane and load
    for (int k = lane * 8; k < d; k += 256) {
      float w8[8];
      unpack8(ld_16B(wr + k), w8);
      const float4 x0 = *reinterpret_cast<const float4*>(xr + k), x1 = *reinterpret_cast<const float4*>(xr + k + 4);
      acc = fmaf(w8[0], x0.x, acc); acc = fmaf(w8[1], x0.y, acc); acc = fmaf(w8[2], x0.z, acc); acc = fmaf(w8[3], x0.w, acc);
      acc = fmaf(w8[4], x1.x, acc); acc = fmaf(w8[5], x1.y, acc); acc = fmaf(w8[6], x1.z, acc); acc = fmaf(w8[7], x1.w, acc);
    }
  } else {
    for (int k = lane; k < d; k += 32) acc = fmaf(to_f(wr[k]), xr[k], acc);
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    int id = ids[row];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    g[row * n + c] = from_f<E>(gelu_new_f(acc) * to_f(table[(size_t)id * ld_tab + off + c]));
  }
}
}  // namespace dli

using namespace dli;

#define DT_CHECK(dt) DLI_CHECK_ARG((dt) == 0 || (dt) == 1, "element type %d: 0 = bf16, 1 = float", dt)

// few rows of a wide model: one CTA per row needs many threads to cover the row's latency; many rows: 256 are enough
static inline int row_threads(int rows, int d) { return (rows <= 64 && d >= 2048) ? 1024 : 256; }

extern "C" {

int dli_embedding_f32(const int32_t* ids, const void* table, float* x, float* x2, void* xe, int rows, int d, int vocab,
                      float scale, int dt, const int32_t* row_ent, const int32_t* ent, const float* inv_freq,
                      dli_stream_t stream) {
  DLI_CHECK_ARG(ids && table && x && d > 0 && vocab > 0, "dli_embedding_f32: null pointer or empty shape");
  DLI_CHECK_ARG(!inv_freq || (row_ent && ent && (reinterpret_cast<uintptr_t>(ent) & 15u) == 0),
                "dli_embedding_f32: positions need row_ent and a 16-byte aligned ent");
  DT_CHECK(dt);
  if (rows <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dt == 0) DLI_LAUNCH("embedding_f32", embedding_f32_kernel<bf16>, dim3(rows), dim3(row_threads(rows, d)), 0, s, ids, (const bf16*)table, x, x2, (bf16*)xe, d, vocab, scale, row_ent, ent, inv_freq);
  else DLI_LAUNCH("embedding_f32", embedding_f32_kernel<float>, dim3(rows), dim3(row_threads(rows, d)), 0, s, ids, (const float*)table, x, x2, (float*)xe, d, vocab, scale, row_ent, ent, inv_freq);
  return DLI_OK;
}

int dli_group_rmsnorm(const float* x, const float* w, float* hn, void* he, int rows, int d, int groups, float eps, int dt,
                      dli_stream_t stream) {
  DLI_CHECK_ARG(x && w && (hn || he) && d > 0 && groups > 0 && d % groups == 0,
                "dli_group_rmsnorm: null pointer, or width %d is not a multiple of %d groups", d, groups);
  DT_CHECK(dt);
  if (rows <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int th = (rows <= 64 && d / groups >= 2048) ? 1024 : 256;
  if (dt == 0) DLI_LAUNCH("group_rmsnorm", group_rmsnorm_kernel<bf16>, dim3(rows), dim3(th), 0, s, x, w, hn, (bf16*)he, d, groups, eps);
  else DLI_LAUNCH("group_rmsnorm", group_rmsnorm_kernel<float>, dim3(rows), dim3(th), 0, s, x, w, hn, (float*)he, d, groups, eps);
  return DLI_OK;
}

int dli_group_rmsnorm_conv_single(const float* x, const float* w, float* hn, void* he, float* tail, const float* conv_w,
                                  const int32_t* ent, void* hc, int rows, int d, int groups, float eps, int taps, int dt,
                                  dli_stream_t stream) {
  DLI_CHECK_ARG(x && w && conv_w && ent && hc && d > 0 && groups > 0 && groups <= kMaxNormGroups && d % groups == 0 &&
                    taps >= 1 && (tail || taps == 1),
                "dli_group_rmsnorm_conv_single: null pointer, or width %d / groups %d (<= %d) / taps %d", d, groups,
                kMaxNormGroups, taps);
  DLI_CHECK_ARG((reinterpret_cast<uintptr_t>(ent) & 15u) == 0, "dli_group_rmsnorm_conv_single: ent must be 16-byte aligned");
  DT_CHECK(dt);
  if (rows <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int th = d >= 2048 ? 1024 : 256;
  if (dt == 0) DLI_LAUNCH("group_rmsnorm_conv_single", group_rmsnorm_conv_single_kernel<bf16>, dim3(rows), dim3(th), 0, s, x, w, hn, (bf16*)he, tail, conv_w, ent, (bf16*)hc, d, groups, eps, taps);
  else DLI_LAUNCH("group_rmsnorm_conv_single", group_rmsnorm_conv_single_kernel<float>, dim3(rows), dim3(th), 0, s, x, w, hn, (float*)he, tail, conv_w, ent, (float*)hc, d, groups, eps, taps);
  return DLI_OK;
}

int dli_residual_add2(float* x, const void* y1, const void* y2, const float* a, const float* h, int rows, int d, int dt,
                      dli_stream_t stream) {
  DLI_CHECK_ARG(x && y1 && d > 0 && (!a || h), "dli_residual_add2: null pointer or empty shape");
  DT_CHECK(dt);
  if (rows <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int gy = rows <= 64 ? (d + 1023) / 1024 : 1;
  if (dt == 0) DLI_LAUNCH("residual_add2", residual_add2_kernel<bf16>, dim3(rows, gy), dim3(256), 0, s, x, (const bf16*)y1, (const bf16*)y2, a, h, d);
  else DLI_LAUNCH("residual_add2", residual_add2_kernel<float>, dim3(rows, gy), dim3(256), 0, s, x, (const float*)y1, (const float*)y2, a, h, d);
  return DLI_OK;
}

int dli_concat_cast(const float* a, const float* b, void* out, int rows, int d, int dt, dli_stream_t stream) {
  DLI_CHECK_ARG(a && b && out && d > 0, "dli_concat_cast: null pointer or empty shape");
  DT_CHECK(dt);
  if (rows <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dt == 0) DLI_LAUNCH("concat_cast", concat_cast_kernel<bf16>, dim3(rows), dim3(256), 0, s, a, b, (bf16*)out, d);
  else DLI_LAUNCH("concat_cast", concat_cast_kernel<float>, dim3(rows), dim3(256), 0, s, a, b, (float*)out, d);
  return DLI_OK;
}

int dli_rows_bias_f32(const void* y, const float* bias, float* x, int rows, int d, int dt, dli_stream_t stream) {
  DLI_CHECK_ARG(y && x && d > 0, "dli_rows_bias_f32: null pointer or empty shape");
  DT_CHECK(dt);
  if (rows <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dt == 0) DLI_LAUNCH("rows_bias_f32", rows_bias_f32_kernel<bf16>, dim3(rows), dim3(256), 0, s, (const bf16*)y, bias, x, d);
  else DLI_LAUNCH("rows_bias_f32", rows_bias_f32_kernel<float>, dim3(rows), dim3(256), 0, s, (const float*)y, bias, x, d);
  return DLI_OK;
}

int dli_scalar_rmsnorm_f32(const float* x, float* hn, int rows, int d, float eps, float g, dli_stream_t stream) {
  DLI_CHECK_ARG(x && hn && d > 0, "dli_scalar_rmsnorm_f32: null pointer or empty shape");
  if (rows <= 0) return DLI_OK;
  DLI_LAUNCH("scalar_rmsnorm", scalar_rmsnorm_kernel, dim3(rows), dim3(row_threads(rows, d)), 0, static_cast<cudaStream_t>(stream), x, hn, d, eps, g);
  return DLI_OK;
}

int dli_postnorm_add_norm(const void* y, float* x, float* hn, int rows, int d, float eps, float g_post, float g_next,
                          int dt, dli_stream_t stream) {
  DLI_CHECK_ARG(y && x && d > 0, "dli_postnorm_add_norm: null pointer or empty shape");
  DT_CHECK(dt);
  if (rows <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dt == 0) DLI_LAUNCH("postnorm_add_norm", postnorm_add_norm_kernel<bf16>, dim3(rows), dim3(row_threads(rows, d)), 0, s, (const bf16*)y, x, hn, d, eps, g_post, g_next);
  else DLI_LAUNCH("postnorm_add_norm", postnorm_add_norm_kernel<float>, dim3(rows), dim3(row_threads(rows, d)), 0, s, (const float*)y, x, hn, d, eps, g_post, g_next);
  return DLI_OK;
}

int dli_causal_conv_ragged(const float* h, float* tail, const float* w, const int32_t* row_ent, const int32_t* ent,
                           void* out, int rows, int n_ent, int d, int taps, int dt, dli_stream_t stream) {
  DLI_CHECK_ARG(h && w && row_ent && ent && out && d > 0 && taps >= 1, "dli_causal_conv_ragged: null pointer or empty shape");
  DLI_CHECK_ARG(tail || taps == 1, "dli_causal_conv_ragged: taps > 1 needs a tail state");
  DLI_CHECK_ARG((reinterpret_cast<uintptr_t>(ent) & 15u) == 0, "dli_causal_conv_ragged: ent must be 16-byte aligned");
  DT_CHECK(dt);
  if (rows <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (rows == n_ent && taps > 1) {  // one row per entry
    if (dt == 0) DLI_LAUNCH("causal_conv_single", causal_conv_single_kernel<bf16>, dim3(rows), dim3(256), 0, s, h, tail, w, ent, (bf16*)out, d, taps);
    else DLI_LAUNCH("causal_conv_single", causal_conv_single_kernel<float>, dim3(rows), dim3(256), 0, s, h, tail, w, ent, (float*)out, d, taps);
    return DLI_OK;
  }
  if (dt == 0) DLI_LAUNCH("causal_conv", causal_conv_kernel<bf16>, dim3(rows), dim3(256), 0, s, h, (const float*)tail, w, row_ent, ent, (bf16*)out, d, taps);
  else DLI_LAUNCH("causal_conv", causal_conv_kernel<float>, dim3(rows), dim3(256), 0, s, h, (const float*)tail, w, row_ent, ent, (float*)out, d, taps);
  if (taps > 1) DLI_LAUNCH("conv_tail_update", conv_tail_update_kernel, dim3(n_ent), dim3(256), 0, s, h, tail, ent, d, taps);
  return DLI_OK;
}

int dli_postnorm_add_norm_conv_single(const void* y, float* x, float* tail, const float* w, const int32_t* ent, void* out,
                                      int rows, int d, int taps, float eps, float g_post, float g_next, int dt,
                                      dli_stream_t stream) {
  DLI_CHECK_ARG(x && w && ent && out && d > 0 && taps >= 1 && (tail || taps == 1), "dli_postnorm_add_norm_conv_single: null pointer or empty shape");
  DLI_CHECK_ARG((reinterpret_cast<uintptr_t>(ent) & 15u) == 0, "dli_postnorm_add_norm_conv_single: ent must be 16-byte aligned");
  DT_CHECK(dt);
  if (rows <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dt == 0) DLI_LAUNCH("postnorm_add_norm_conv_single", postnorm_add_norm_conv_single_kernel<bf16>, dim3(rows), dim3(row_threads(rows, d)), 0, s, (const bf16*)y, x, tail, w, ent, (bf16*)out, d, taps, eps, g_post, g_next);
  else DLI_LAUNCH("postnorm_add_norm_conv_single", postnorm_add_norm_conv_single_kernel<float>, dim3(rows), dim3(row_threads(rows, d)), 0, s, (const float*)y, x, tail, w, ent, (float*)out, d, taps, eps, g_post, g_next);
  return DLI_OK;
}

int dli_gather_cast(const float* src, const int32_t* rows, void* out, int n, int d, int dt, dli_stream_t stream) {
  DLI_CHECK_ARG(src && rows && out && d > 0, "dli_gather_cast: null pointer or empty shape");
  DT_CHECK(dt);
  if (n <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dt == 0) DLI_LAUNCH("gather_cast", gather_cast_kernel<bf16>, dim3(n), dim3(256), 0, s, src, rows, (bf16*)out, d);
  else DLI_LAUNCH("gather_cast", gather_cast_kernel<float>, dim3(n), dim3(256), 0, s, src, rows, (float*)out, d);
  return DLI_OK;
}

int dli_linear_any(const void* x, const void* w, void* y, int M, int N, int K, int ldx, int ldy, int dt,
                   dli_stream_t stream) {
  DLI_CHECK_ARG(x && w && y && N > 0 && K > 0 && ldx >= K && ldy >= N, "dli_linear_any: null pointer or bad shape");
  DT_CHECK(dt);
  if (M <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid((N + 63) / 64, (M + 63) / 64);
  if (dt == 0) DLI_LAUNCH("linear_any", linear_any_kernel<bf16, bf16>, grid, dim3(256), 0, s, (const bf16*)x, (const bf16*)w, (bf16*)y, M, N, K, ldx, ldy);
  else DLI_LAUNCH("linear_any", linear_any_kernel<float, float>, grid, dim3(256), 0, s, (const float*)x, (const float*)w, (float*)y, M, N, K, ldx, ldy);
  return DLI_OK;
}

int dli_silu_mul(const void* gu, void* act, int M, int F, int ld, int dt, const float* bias, dli_stream_t stream) {
  DLI_CHECK_ARG(gu && act && F > 0 && ld >= 2 * F, "dli_silu_mul: null pointer or bad shape");
  DT_CHECK(dt);
  if (M <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int per = dt == 0 ? 8 : 4;
  const int vec = F % per == 0 && ld % per == 0 && aligned16(gu) && aligned16(act);
  const int work = F / (vec ? per : 1);
  const dim3 grid(M, M <= 64 ? (work + 1023) / 1024 : (work >= 2048 ? 2 : 1));  // few or long rows: a row's channels go to several CTAs
  if (dt == 0) DLI_LAUNCH("silu_mul", silu_mul_kernel<bf16>, grid, dim3(256), 0, s, (const bf16*)gu, (bf16*)act, F, ld, bias, vec);
  else DLI_LAUNCH("silu_mul", silu_mul_kernel<float>, grid, dim3(256), 0, s, (const float*)gu, (float*)act, F, ld, bias, vec);
  return DLI_OK;
}

int dli_postnorm_vec_add(const void* y, float* x, const float* w, void* he, int rows, int d, float eps, int dt,
                         dli_stream_t stream) {
  DLI_CHECK_ARG(x && d > 0 && (y == nullptr || w) && (y || he), "dli_postnorm_vec_add: null pointer or empty shape");
  DT_CHECK(dt);
  if (rows <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dt == 0) DLI_LAUNCH("postnorm_vec_add", postnorm_vec_add_kernel<bf16>, dim3(rows), dim3(row_threads(rows, d)), 0, s, (const bf16*)y, x, w, (bf16*)he, d, eps);
  else DLI_LAUNCH("postnorm_vec_add", postnorm_vec_add_kernel<float>, dim3(rows), dim3(row_threads(rows, d)), 0, s, (const float*)y, x, w, (float*)he, d, eps);
  return DLI_OK;
}

int dli_token_side_act(const void* s_in, const int32_t* ids, const void* table, void* g, int rows, int n, int ld_tab, int off,
                       int vocab, int dt, dli_stream_t stream) {
  DLI_CHECK_ARG(s_in && ids && table && g && n > 0 && off >= 0 && off + n <= ld_tab && vocab > 0,
                "dli_token_side_act: null pointer or bad shape");
  DT_CHECK(dt);
  if (rows <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dt == 0) DLI_LAUNCH("token_side_act", token_side_act_kernel<bf16>, dim3(rows), dim3(n <= 128 ? 128 : 256), 0, s, (const bf16*)s_in, ids, (const bf16*)table, (bf16*)g, n, ld_tab, off, vocab);
  else DLI_LAUNCH("token_side_act", token_side_act_kernel<float>, dim3(rows), dim3(n <= 128 ? 128 : 256), 0, s, (const float*)s_in, ids, (const float*)table, (float*)g, n, ld_tab, off, vocab);
  return DLI_OK;
}

int dli_token_side(float* x, const int32_t* ids, const void* table, const void* w_gate, const void* w_proj, const float* w,
                   void* he, int rows, int d, int n, int ld_tab, int off, int vocab, float eps, int dt, dli_stream_t stream) {
  DLI_CHECK_ARG(x && ids && table && w_gate && w_proj && w && d > 0 && n > 0 && off >= 0 && off + n <= ld_tab && vocab > 0,
                "dli_token_side: null pointer or bad shape");
  const size_t smem = sizeof(float) * (2 * (size_t)d + n);
  DLI_CHECK_ARG(smem <= 48 * 1024, "dli_token_side: width %d with %d side channels needs %zu bytes of shared memory", d, n, smem);
  DT_CHECK(dt);
  if (rows <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int th = d >= 2048 ? 1024 : (d >= 512 ? 512 : 256);
  if (dt == 0) DLI_LAUNCH("token_side", token_side_kernel<bf16>, dim3(rows), dim3(th), smem, s, x, ids, (const bf16*)table, (const bf16*)w_gate, (const bf16*)w_proj, w, (bf16*)he, d, n, ld_tab, off, vocab, eps);
  else DLI_LAUNCH("token_side", token_side_kernel<float>, dim3(rows), dim3(th), smem, s, x, ids, (const float*)table, (const float*)w_gate, (const float*)w_proj, w, (float*)he, d, n, ld_tab, off, vocab, eps);
  return DLI_OK;
}


int dli_token_side_gate(const float* x, const int32_t* ids, const void* table, const void* w_gate, void* g, int rows, int d,
                        int n, int ld_tab, int off, int vocab, int dt, dli_stream_t stream) {
  DLI_CHECK_ARG(x && ids && table && w_gate && g && d > 0 && n > 0 && off >= 0 && off + n <= ld_tab && vocab > 0,
                "dli_token_side_gate: null pointer or bad shape");
  DT_CHECK(dt);
  if (rows <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(rows, (n + 7) / 8);
  if (dt == 0) DLI_LAUNCH("token_side_gate", token_side_gate_kernel<bf16>, grid, dim3(256), 0, s, x, ids, (const bf16*)table, (const bf16*)w_gate, (bf16*)g, d, n, ld_tab, off, vocab);
  else DLI_LAUNCH("token_side_gate", token_side_gate_kernel<float>, grid, dim3(256), 0, s, x, ids, (const float*)table, (const float*)w_gate, (float*)g, d, n, ld_tab, off, vocab);
  return DLI_OK;
}

}  // extern "C"
