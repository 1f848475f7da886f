// Gated delta-rule mixer for a RAGGED step.  Per value head h (its queries and keys come from head h / (H/G) of the
// G query/key heads) the layer keeps a matrix S [D, V] per sequence:
//   q_t, k_t  unit vectors (x / sqrt(sum x^2 + unit_eps)), q_t also times q_scale
//   beta_t = sigmoid(b_t),  g_t = exp(-exp(A_log_h) * softplus(a_t + dt_bias_h))
//   S <- g_t S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t      (the read-out sees the write)
// Column c of S (all D rows of one value dimension) never meets another column, so the recurrence is dealt to the
// GPU by value column: a warp owns kDeltaCols columns with lane l holding rows l, l + 32, ... in registers, a CTA
// owns 8 warps' columns of one (entry, head) and walks the entry's rows in order.  The rows' q, k (normalised once
// per CTA), v, beta and g are staged in shared memory kDeltaBlock rows at a time.  The state is stored value-major,
// S^T [slots, H, V, D], so that a warp reads and writes its columns as contiguous runs.
//   dli_delta_rule_ragged   qkv fp32 [rows, 2*G*D + H*V] (q | k | v after their convolutions and activations),
//                           b_t / a_t columns of the projection row -> o fp32 [rows, H*V]; state read and advanced
//   dli_head_rmsnorm_gate   out[row, h, :] = o / sqrt(mean(o^2) + eps) * w * act(gate[row, h, :])
// Everything is fp32 except the projection row (b, a, gate) and the output, which have the engine's element type.
// An entry whose first position is 0 starts from a zero state whatever its slot held before.
#include <math.h>

#include "common.cuh"

namespace dli {

template <typename E> __device__ __forceinline__ float d_to_f(E v);
template <> __device__ __forceinline__ float d_to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float d_to_f<bf16>(bf16 v) { return __bfloat162float(v); }
template <typename E> __device__ __forceinline__ E d_from_f(float v);
template <> __device__ __forceinline__ float d_from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 d_from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

struct DeltaRun {
  const int32_t* ent;
  int H, G, D, V;
  int ldx;                  // row stride of qkv
  int ldp, b_off, a_off;    // projection row: stride, column of beta's and of the decay's pre-activation (per head)
  const float* a_log;       // [H]
  const float* dt_bias;     // [H]
  float q_scale, unit_eps;
};

constexpr int kDeltaWarps = 8;
constexpr int kDeltaCols = 2;    // value columns per warp
constexpr int kDeltaBlock = 16;  // rows staged per pass

// Grid (entries, H, ceil(V / (kDeltaWarps * kDeltaCols))).  NS = ceil(D / 32) state rows per lane and column.
template <typename E, int NS>
__global__ void __launch_bounds__(kDeltaWarps * 32)
delta_rule_kernel(const float* __restrict__ qkv, const E* __restrict__ proj, float* __restrict__ St,
                  float* __restrict__ o, DeltaRun a) {
  extern __shared__ float sm_delta[];
  const int D = a.D;
  float* qs = sm_delta;                                    // [kDeltaBlock][D]
  float* ks = qs + kDeltaBlock * D;                        // [kDeltaBlock][D]
  float* vs = ks + kDeltaBlock * D;                        // [kDeltaBlock][kDeltaWarps * kDeltaCols]
  float* bg = vs + kDeltaBlock * kDeltaWarps * kDeltaCols; // [kDeltaBlock][2]: beta, g
  pdl_wait();
  pdl_trigger();
  const int4 e = reinterpret_cast<const int4*>(a.ent)[blockIdx.x];  // slot, first row, rows, first position
  const int h = blockIdx.y, gq = h / (a.H / a.G);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int CPB = kDeltaWarps * kDeltaCols;
  const int c0 = blockIdx.z * CPB + warp * kDeltaCols;
  float s[kDeltaCols][NS];
#pragma unroll
  for (int c = 0; c < kDeltaCols; ++c) {
    const float* sp = St + (((size_t)e.x * a.H + h) * a.V + (c0 + c)) * D;
#pragma unroll
    for (int n = 0; n < NS; ++n) {
      const int i = lane + 32 * n;
      s[c][n] = (e.w > 0 && c0 + c < a.V && i < D) ? sp[i] : 0.f;
    }
  }
  const float neg_a = -expf(a.a_log[h]), dtb = a.dt_bias[h];
  const int q_col = gq * D, k_col = a.G * D + gq * D, v_col = 2 * a.G * D + h * a.V + blockIdx.z * CPB;

  for (int t0 = 0; t0 < e.z; t0 += kDeltaBlock) {
    const int nt = min(kDeltaBlock, e.z - t0);
    __syncthreads();  // the previous pass has been consumed
    // a warp normalises the queries and keys of rows warp, warp + 8, ...
    for (int t = warp; t < nt; t += kDeltaWarps) {
      const float* xr = qkv + (size_t)(e.y + t0 + t) * a.ldx;
      float qv[NS], kv[NS], qq = 0.f, kk = 0.f;
#pragma unroll
      for (int n = 0; n < NS; ++n) {
        const int i = lane + 32 * n;
        qv[n] = i < D ? xr[q_col + i] : 0.f;
        kv[n] = i < D ? xr[k_col + i] : 0.f;
        qq = fmaf(qv[n], qv[n], qq);
        kk = fmaf(kv[n], kv[n], kk);
      }
      qq = a.q_scale / sqrtf(warp_sum(qq) + a.unit_eps);
      kk = 1.f / sqrtf(warp_sum(kk) + a.unit_eps);
#pragma unroll
      for (int n = 0; n < NS; ++n) {
        const int i = lane + 32 * n;
        if (i < D) { qs[t * D + i] = qv[n] * qq; ks[t * D + i] = kv[n] * kk; }
      }
    }
    for (int i = tid; i < nt * CPB; i += kDeltaWarps * 32) {
      const int t = i / CPB, c = i - t * CPB;
      vs[i] = (blockIdx.z * CPB + c < a.V) ? qkv[(size_t)(e.y + t0 + t) * a.ldx + v_col + c] : 0.f;
    }
    if (tid < nt) {
      const E* pr = proj + (size_t)(e.y + t0 + tid) * a.ldp;
      const float b = d_to_f(pr[a.b_off + h]), x = d_to_f(pr[a.a_off + h]) + dtb;
      const float sp = x > 20.f ? x : log1pf(expf(x));
      bg[2 * tid] = 1.f / (1.f + expf(-b));
      bg[2 * tid + 1] = expf(neg_a * sp);
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      float kk[NS], qq[NS];
#pragma unroll
      for (int n = 0; n < NS; ++n) {
        const int i = lane + 32 * n;
        kk[n] = i < D ? ks[t * D + i] : 0.f;
        qq[n] = i < D ? qs[t * D + i] : 0.f;
      }
      const float beta = bg[2 * t], g = bg[2 * t + 1];
      float r[kDeltaCols];
#pragma unroll
      for (int c = 0; c < kDeltaCols; ++c) {
        r[c] = 0.f;
#pragma unroll
        for (int n = 0; n < NS; ++n) r[c] = fmaf(s[c][n], kk[n], r[c]);
      }
#pragma unroll
      for (int c = 0; c < kDeltaCols; ++c) r[c] = warp_sum(r[c]);
      float ov[kDeltaCols];
#pragma unroll
      for (int c = 0; c < kDeltaCols; ++c) {
        const float u = beta * (vs[t * CPB + warp * kDeltaCols + c] - g * r[c]);
        ov[c] = 0.f;
#pragma unroll
        for (int n = 0; n < NS; ++n) {
          s[c][n] = fmaf(g, s[c][n], kk[n] * u);
          ov[c] = fmaf(s[c][n], qq[n], ov[c]);
        }
      }
#pragma unroll
      for (int c = 0; c < kDeltaCols; ++c) ov[c] = warp_sum(ov[c]);
      if (lane < kDeltaCols && c0 + lane < a.V) {
        float val = ov[0];
#pragma unroll
        for (int c = 1; c < kDeltaCols; ++c) if (lane == c) val = ov[c];
        o[(size_t)(e.y + t0 + t) * (a.H * a.V) + h * a.V + c0 + lane] = val;
      }
    }
  }
#pragma unroll
  for (int c = 0; c < kDeltaCols; ++c) {
    if (c0 + c >= a.V) continue;
    float* sp = St + (((size_t)e.x * a.H + h) * a.V + (c0 + c)) * D;
#pragma unroll
    for (int n = 0; n < NS; ++n) {
      const int i = lane + 32 * n;
      if (i < D) sp[i] = s[c][n];
    }
  }
}

// One warp per (row, head): RMS norm over the head's V outputs, weight, gate.  w_heads != 0: w is [H, V], else [V]
// shared by the heads.  gate: 0 none, 1 SiLU, 2 sigmoid of proj[row, g_off + h*V + v].
template <typename E>
__global__ void __launch_bounds__(256)
head_rmsnorm_gate_kernel(const float* __restrict__ o, const E* __restrict__ proj, const float* __restrict__ w,
                         E* __restrict__ out, int rows, int H, int V, float eps, int w_heads, int gate, int ldp,
                         int g_off) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const size_t item = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (size_t)rows * H) return;
  const size_t row = item / H;
  const int h = (int)(item - row * H);
  const float* src = o + item * V;
  float ss = 0.f;
  for (int v = lane; v < V; v += 32) ss = fmaf(src[v], src[v], ss);
  const float r = 1.f / sqrtf(warp_sum(ss) / V + eps);
  for (int v = lane; v < V; v += 32) {
    float y = src[v] * r * w[w_heads ? h * V + v : v];
    if (gate) {
      const float z = d_to_f(proj[row * ldp + g_off + h * V + v]);
      y *= gate == 1 ? z / (1.f + expf(-z)) : 1.f / (1.f + expf(-z));
    }
    out[item * V + v] = d_from_f<E>(y);
  }
}

template <typename E, int NS>
static int launch_delta(const float* qkv, const void* proj, float* St, float* o, int n_ent, const DeltaRun& a,
                        cudaStream_t s) {
  const size_t smem = sizeof(float) * ((size_t)2 * kDeltaBlock * a.D + kDeltaBlock * kDeltaWarps * kDeltaCols + 2 * kDeltaBlock);
  const dim3 grid(n_ent, a.H, (a.V + kDeltaWarps * kDeltaCols - 1) / (kDeltaWarps * kDeltaCols));
  DLI_LAUNCH("delta_rule", (delta_rule_kernel<E, NS>), grid, dim3(kDeltaWarps * 32), smem, s, qkv, (const E*)proj, St, o, a);
  return DLI_OK;
}

template <typename E>
static int dispatch_delta(const float* qkv, const void* proj, float* St, float* o, int n_ent, const DeltaRun& a,
                          cudaStream_t s) {
  if (a.D <= 32) return launch_delta<E, 1>(qkv, proj, St, o, n_ent, a, s);
  if (a.D <= 64) return launch_delta<E, 2>(qkv, proj, St, o, n_ent, a, s);
  if (a.D <= 128) return launch_delta<E, 4>(qkv, proj, St, o, n_ent, a, s);
  return launch_delta<E, 8>(qkv, proj, St, o, n_ent, a, s);
}

}  // namespace dli

using namespace dli;

extern "C" {

int dli_delta_rule_ragged(const float* qkv, const void* proj, float* St, float* o, const int32_t* ent, int n_ent, int H,
                          int G, int D, int V, int ldx, int ldp, int b_off, int a_off, const float* a_log,
                          const float* dt_bias, float q_scale, float unit_eps, int dt, dli_stream_t stream) {
  DLI_CHECK_ARG(qkv && proj && St && o && ent && a_log && dt_bias, "dli_delta_rule_ragged: null pointer");
  DLI_CHECK_ARG(H > 0 && G > 0 && H % G == 0 && D > 0 && D <= 256 && V > 0 && ldx >= 2 * G * D + H * V,
                "dli_delta_rule_ragged: H=%d G=%d D=%d V=%d ldx=%d (H %% G == 0, D <= 256)", H, G, D, V, ldx);
  DLI_CHECK_ARG((reinterpret_cast<uintptr_t>(ent) & 15u) == 0, "dli_delta_rule_ragged: ent must be 16-byte aligned");
  DLI_CHECK_ARG(dt == 0 || dt == 1, "element type %d: 0 = bf16, 1 = float", dt);
  if (n_ent <= 0) return DLI_OK;
  DeltaRun a{ent, H, G, D, V, ldx, ldp, b_off, a_off, a_log, dt_bias, q_scale, unit_eps};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return dt == 0 ? dispatch_delta<bf16>(qkv, proj, St, o, n_ent, a, s) : dispatch_delta<float>(qkv, proj, St, o, n_ent, a, s);
}

int dli_head_rmsnorm_gate(const float* o, const void* proj, const float* w, void* out, int rows, int H, int V, float eps,
                          int w_heads, int gate, int ldp, int g_off, int dt, dli_stream_t stream) {
  DLI_CHECK_ARG(o && w && out && (gate == 0 || proj) && gate >= 0 && gate <= 2 && H > 0 && V > 0,
                "dli_head_rmsnorm_gate: null pointer or bad shape");
  DLI_CHECK_ARG(dt == 0 || dt == 1, "element type %d: 0 = bf16, 1 = float", dt);
  if (rows <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)(((size_t)rows * H + 7) / 8);
  if (dt == 0) DLI_LAUNCH("head_rmsnorm_gate", head_rmsnorm_gate_kernel<bf16>, dim3(grid), dim3(256), 0, s, o, (const bf16*)proj, w, (bf16*)out, rows, H, V, eps, w_heads, gate, ldp, g_off);
  else DLI_LAUNCH("head_rmsnorm_gate", head_rmsnorm_gate_kernel<float>, dim3(grid), dim3(256), 0, s, o, (const float*)proj, w, (float*)out, rows, H, V, eps, w_heads, gate, ldp, g_off);
  return DLI_OK;
}

}  // extern "C"
