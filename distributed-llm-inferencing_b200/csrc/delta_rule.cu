// Gated delta-rule mixer for a RAGGED step.  Per value head h (its queries and keys come from head h / (H/G) of the
// G query/key heads) the layer keeps a matrix S [D, V] per sequence:
//   q_t, k_t  unit vectors (x / sqrt(sum x^2 + unit_eps)), q_t also times q_scale
//   beta_t = sigmoid(b_t),  g_t = exp(-exp(A_log_h) * softplus(a_t + dt_bias_h))
//   S <- g_t S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t      (the read-out sees the write:
//   o_t = g_t S_(t-1)^T q_t + u (k_t . q_t), which is how the kernel evaluates it)
// Column c of S (all D rows of one value dimension) never meets another column, so the recurrence is dealt to the
// GPU by value column: a column's D rows live in the registers of consecutive lanes (4, 8 or 16 rows each), a thread
// carries one or two columns, and a CTA of 4 warps walks the rows of one (entry, head) in order.  The rows' q, k (normalised
// once per CTA), v, beta and g are staged in shared memory kDeltaBlock rows at a time.  The state is stored value-major,
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

constexpr int kDeltaWarps = 4;
constexpr int kDeltaBlock = 16;  // rows of the step staged per pass
// NS state rows per thread and column: 16 or 8 (a lane's key entries start NS + 4 floats apart, which spreads its
// 16-byte loads over the banks) or 4 (a warp's lanes read 512 consecutive bytes)
__host__ __device__ constexpr int delta_pad(int NS) { return NS == 4 ? 4 : NS + 4; }
constexpr int kDeltaPre = 4;     // a lane prefetches up to 4 query and 4 key entries of a row (key sizes up to 128)

// lanes that share a column: the smallest power of two with lanes * NS >= D
__host__ __device__ inline int delta_lanes(int D, int NS) {
  int l = 1;
  while (l * NS < D) l <<= 1;
  return l;
}
__host__ __device__ inline int delta_cols_per_cta(int D, int NS, int cpt) { return kDeltaWarps * (32 / delta_lanes(D, NS)) * cpt; }

// Grid (entries, H, ceil(V / columns per CTA)).  A column's D state rows are dealt to `lanes` consecutive lanes, NS
// consecutive rows each, so S^T k and S^T q need NS multiply-adds and log2(lanes) shuffles per lane; a thread carries
// CPT columns.  The walk over the rows is one dependent chain per column, so its speed is set by how many warps a
// scheduler can switch between: (NS, CPT) = (16, 2) does the work with the fewest instructions and is taken when
// there are columns enough to fill the GPU with it, (16, 1), (8, 1) and (4, 1) spread the same columns over 2x, 4x and
// 8x as many warps.  While a pass of 16 rows is computed, the next pass's raw q and k rows are already on their way
// into registers (key sizes up to 128), so the recurrence does not wait for global memory between passes.
template <typename E, int CPT, int NS>
__global__ void __launch_bounds__(kDeltaWarps * 32)
delta_rule_kernel(const float* __restrict__ qkv, const E* __restrict__ proj, float* __restrict__ St,
                  float* __restrict__ o, DeltaRun a) {
  extern __shared__ __align__(16) float sm_delta[];
  constexpr int kDeltaRows = NS, kDeltaPad = delta_pad(NS);
  const int D = a.D, lanes = delta_lanes(D, NS), ldk = lanes * kDeltaPad, cpb = delta_cols_per_cta(D, NS, CPT);
  float* qs = sm_delta;                   // [kDeltaBlock][ldk]
  float* ks = qs + kDeltaBlock * ldk;     // [kDeltaBlock][ldk]
  float* vs = ks + kDeltaBlock * ldk;     // [kDeltaBlock][cpb]
  float* bg = vs + kDeltaBlock * cpb;     // [kDeltaBlock][3]: beta, g, k . q of the unit vectors (q scaled)
  pdl_wait();
  pdl_trigger();
  const int4 e = reinterpret_cast<const int4*>(a.ent)[blockIdx.x];  // slot, first row, rows, first position
  const int h = blockIdx.y, gq = h / (a.H / a.G);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int p = lane % lanes, cg = lane / lanes;             // part of the column, column group within the warp
  const int cl = (warp * (32 / lanes) + cg) * CPT;           // first of the thread's columns within the CTA
  const int c0 = blockIdx.z * cpb + cl;
  const int r0 = p * kDeltaRows;                             // the thread's first state row
  float s[CPT][kDeltaRows];
#pragma unroll
  for (int c = 0; c < CPT; ++c) {
    const float* sp = St + (((size_t)e.x * a.H + h) * a.V + (c0 + c)) * D + r0;
#pragma unroll
    for (int n = 0; n < kDeltaRows; ++n) s[c][n] = (e.w > 0 && c0 + c < a.V && r0 + n < D) ? sp[n] : 0.f;
  }
  const float neg_a = -expf(a.a_log[h]), dtb = a.dt_bias[h];
  const int q_col = gq * D, k_col = a.G * D + gq * D, v_col = 2 * a.G * D + h * a.V + blockIdx.z * cpb;
  const bool pre = D <= 32 * kDeltaPre;
  constexpr int TPW = kDeltaBlock / kDeltaWarps;             // rows of a pass that one warp normalises
  float pq[TPW][kDeltaPre], pk[TPW][kDeltaPre];

  // raw q and k entries of the warp's rows of the pass that starts at row t0 -> registers
  auto fetch = [&](int t0) {
    const int nt = min(kDeltaBlock, e.z - t0);
#pragma unroll
    for (int j = 0; j < TPW; ++j) {
      const int t = warp + j * kDeltaWarps;
      const float* xr = qkv + (size_t)(e.y + t0 + min(t, nt - 1)) * a.ldx;
#pragma unroll
      for (int n = 0; n < kDeltaPre; ++n) {
        const int i = lane + 32 * n;
        pq[j][n] = i < D ? xr[q_col + i] : 0.f;
        pk[j][n] = i < D ? xr[k_col + i] : 0.f;
      }
    }
  };
  if (pre && e.z > 0) fetch(0);

  for (int t0 = 0; t0 < e.z; t0 += kDeltaBlock) {
    const int nt = min(kDeltaBlock, e.z - t0);
    __syncthreads();  // the previous pass has been consumed
    // a warp normalises the queries and keys of rows warp, warp + 4, ...
    if (pre) {
#pragma unroll
      for (int j = 0; j < TPW; ++j) {
        const int t = warp + j * kDeltaWarps;
        float qq = 0.f, kk = 0.f, qk = 0.f;
#pragma unroll
        for (int n = 0; n < kDeltaPre; ++n) {
          qq = fmaf(pq[j][n], pq[j][n], qq);
          kk = fmaf(pk[j][n], pk[j][n], kk);
          qk = fmaf(pq[j][n], pk[j][n], qk);
        }
        qq = a.q_scale / sqrtf(warp_sum(qq) + a.unit_eps);
        kk = 1.f / sqrtf(warp_sum(kk) + a.unit_eps);
        qk = warp_sum(qk) * qq * kk;
        if (t < nt) {
          if (lane == 0) bg[3 * t + 2] = qk;
#pragma unroll
          for (int n = 0; n < kDeltaPre; ++n) {
            const int i = lane + 32 * n;
            if (i < lanes * kDeltaRows) {
              const int at = t * ldk + (i / kDeltaRows) * kDeltaPad + i % kDeltaRows;
              qs[at] = pq[j][n] * qq;
              ks[at] = pk[j][n] * kk;
            }
          }
        }
      }
    } else {
      for (int t = warp; t < nt; t += kDeltaWarps) {
        const float* xr = qkv + (size_t)(e.y + t0 + t) * a.ldx;
        float qq = 0.f, kk = 0.f, qk = 0.f;
        for (int i = lane; i < D; i += 32) {
          const float qv = xr[q_col + i], kv = xr[k_col + i];
          qq = fmaf(qv, qv, qq);
          kk = fmaf(kv, kv, kk);
          qk = fmaf(qv, kv, qk);
        }
        qq = a.q_scale / sqrtf(warp_sum(qq) + a.unit_eps);
        kk = 1.f / sqrtf(warp_sum(kk) + a.unit_eps);
        qk = warp_sum(qk) * qq * kk;
        if (lane == 0) bg[3 * t + 2] = qk;
        for (int i = lane; i < lanes * kDeltaRows; i += 32) {
          const int at = t * ldk + (i / kDeltaRows) * kDeltaPad + i % kDeltaRows;
          qs[at] = i < D ? xr[q_col + i] * qq : 0.f;
          ks[at] = i < D ? xr[k_col + i] * kk : 0.f;
        }
      }
    }
    for (int i = tid; i < nt * cpb; i += kDeltaWarps * 32) {
      const int t = i / cpb, c = i - t * cpb;
      vs[i] = (blockIdx.z * cpb + c < a.V) ? qkv[(size_t)(e.y + t0 + t) * a.ldx + v_col + c] : 0.f;
    }
    if (tid < nt) {
      const E* pr = proj + (size_t)(e.y + t0 + tid) * a.ldp;
      const float b = d_to_f(pr[a.b_off + h]), x = d_to_f(pr[a.a_off + h]) + dtb;
      const float sp = x > 20.f ? x : log1pf(expf(x));
      bg[3 * tid] = 1.f / (1.f + expf(-b));
      bg[3 * tid + 1] = expf(neg_a * sp);
    }
    __syncthreads();
    if (pre && t0 + kDeltaBlock < e.z) fetch(t0 + kDeltaBlock);   // in flight while this pass is computed
#pragma unroll 4
    for (int t = 0; t < nt; ++t) {
      float kk[kDeltaRows], qq[kDeltaRows];
      const float4* kp = reinterpret_cast<const float4*>(ks + t * ldk + p * kDeltaPad);
      const float4* qp = reinterpret_cast<const float4*>(qs + t * ldk + p * kDeltaPad);
#pragma unroll
      for (int n = 0; n < kDeltaRows / 4; ++n) {
        const float4 kf = kp[n], qf = qp[n];
        kk[4 * n] = kf.x; kk[4 * n + 1] = kf.y; kk[4 * n + 2] = kf.z; kk[4 * n + 3] = kf.w;
        qq[4 * n] = qf.x; qq[4 * n + 1] = qf.y; qq[4 * n + 2] = qf.z; qq[4 * n + 3] = qf.w;
      }
      const float beta = bg[3 * t], g = bg[3 * t + 1], kq = bg[3 * t + 2];
      // both read-outs come from the state BEFORE this row's write: S_old^T k for the write itself and S_old^T q for the
      // output, o = g S_old^T q + u (k . q); the two reductions run side by side and only the first one is on the path
      // to the next row
      float ra[CPT], rb[CPT];
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        float a4[4] = {0.f, 0.f, 0.f, 0.f}, b4[4] = {0.f, 0.f, 0.f, 0.f};   // partial sums: chains of NS / 4 multiply-adds
#pragma unroll
        for (int n = 0; n < kDeltaRows; ++n) {
          a4[n & 3] = fmaf(s[c][n], kk[n], a4[n & 3]);
          b4[n & 3] = fmaf(s[c][n], qq[n], b4[n & 3]);
        }
        ra[c] = (a4[0] + a4[1]) + (a4[2] + a4[3]);
        rb[c] = (b4[0] + b4[1]) + (b4[2] + b4[3]);
      }
      for (int off = 1; off < lanes; off <<= 1) {
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
          ra[c] += __shfl_xor_sync(0xffffffffu, ra[c], off);
          rb[c] += __shfl_xor_sync(0xffffffffu, rb[c], off);
        }
      }
      float ov[CPT];
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        const float u = beta * (vs[t * cpb + cl + c] - g * ra[c]);
        ov[c] = fmaf(g, rb[c], u * kq);
#pragma unroll
        for (int n = 0; n < kDeltaRows; ++n) s[c][n] = fmaf(g, s[c][n], kk[n] * u);
      }
      if (p == 0) {
        float* orow = o + (size_t)(e.y + t0 + t) * (a.H * a.V) + h * a.V + c0;
#pragma unroll
        for (int c = 0; c < CPT; ++c)
          if (c0 + c < a.V) orow[c] = ov[c];
      }
    }
  }
#pragma unroll
  for (int c = 0; c < CPT; ++c) {
    if (c0 + c >= a.V) continue;
    float* sp = St + (((size_t)e.x * a.H + h) * a.V + (c0 + c)) * D + r0;
#pragma unroll
    for (int n = 0; n < kDeltaRows; ++n)
      if (r0 + n < D) sp[n] = s[c][n];
  }
}

// ---- portions of prompts: 16 rows at a time ----------------------------------------------------------------------
// With S the state before a pass of rows t = 0 .. n-1, c_t the running sum of log g, w_t = S^T k_t and z_t = S^T q_t:
//   u_t = beta_t (v_t - e^(c_t) w_t) - sum_(s<t) A[t][s] u_s,      A[t][s] = beta_t e^(c_t - c_s) (k_t . k_s)
//   o_t = e^(c_t) z_t + sum_(s<=t) P[t][s] u_s,                     P[t][s] = e^(c_t - c_s) (q_t . k_s)
//   S  <- e^(c_(n-1)) S + sum_t e^(c_(n-1) - c_t) k_t u_t^T
// (the recurrence above with S_(t-1) written out; every exponent is <= 0).  The 2n read-outs of the old state are
// independent of one another, so their multiply-adds and shuffles overlap instead of forming one chain per row; what
// stays sequential is the n-step substitution for u, a few multiply-adds per step on registers.  A and P are the same for
// all value columns: the CTA forms them once per pass from the staged unit vectors.  Same grid, state layout and staging
// as delta_rule_kernel<E, 1, 16>.
template <typename E>
__global__ void __launch_bounds__(kDeltaWarps * 32)
delta_rule_block_kernel(const float* __restrict__ qkv, const E* __restrict__ proj, float* __restrict__ St,
                        float* __restrict__ o, DeltaRun a) {
  constexpr int NS = 16, kPad = delta_pad(NS), CB = kDeltaBlock;
  extern __shared__ __align__(16) float sm_delta[];
  const int D = a.D, lanes = delta_lanes(D, NS), ldk = lanes * kPad + 4, cpb = delta_cols_per_cta(D, NS, 1);
  float* qs = sm_delta;                 // [CB][ldk]   (rows 4 floats longer than their content: rows of different t
  float* ks = qs + CB * ldk;            // [CB][ldk]    start in different banks for the pairwise products)
  float* vs = ks + CB * ldk;            // [CB][cpb]
  float* bg = vs + CB * cpb;            // [CB][4]: beta, log g, running sum of log g, unused
  float* Am = bg + CB * 4;              // [CB][CB]
  float* Pm = Am + CB * CB;             // [CB][CB]
  pdl_wait();
  pdl_trigger();
  const int4 e = reinterpret_cast<const int4*>(a.ent)[blockIdx.x];
  const int h = blockIdx.y, gq = h / (a.H / a.G);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int p = lane % lanes, cg = lane / lanes;
  const int cl = warp * (32 / lanes) + cg;
  const int c0 = blockIdx.z * cpb + cl;
  const int r0 = p * NS;
  float s[NS];
  {
    const float* sp = St + (((size_t)e.x * a.H + h) * a.V + c0) * D + r0;
#pragma unroll
    for (int n = 0; n < NS; ++n) s[n] = (e.w > 0 && c0 < a.V && r0 + n < D) ? sp[n] : 0.f;
  }
  const float neg_a = -expf(a.a_log[h]), dtb = a.dt_bias[h];
  const int q_col = gq * D, k_col = a.G * D + gq * D, v_col = 2 * a.G * D + h * a.V + blockIdx.z * cpb;
  const bool pre = D <= 32 * kDeltaPre;
  constexpr int TPW = CB / kDeltaWarps;
  float pq[TPW][kDeltaPre], pk[TPW][kDeltaPre];
  auto fetch = [&](int t0) {
    const int nt = min(CB, e.z - t0);
#pragma unroll
    for (int j = 0; j < TPW; ++j) {
      const int t = warp + j * kDeltaWarps;
      const float* xr = qkv + (size_t)(e.y + t0 + min(t, nt - 1)) * a.ldx;
#pragma unroll
      for (int n = 0; n < kDeltaPre; ++n) {
        const int i = lane + 32 * n;
        pq[j][n] = i < D ? xr[q_col + i] : 0.f;
        pk[j][n] = i < D ? xr[k_col + i] : 0.f;
      }
    }
  };
  if (pre && e.z > 0) fetch(0);

  for (int t0 = 0; t0 < e.z; t0 += CB) {
    const int nt = min(CB, e.z - t0);
    __syncthreads();
    // ---- stage the pass: unit q (scaled) and k, v of the CTA's columns, beta and log g
    if (pre) {
#pragma unroll
      for (int j = 0; j < TPW; ++j) {
        const int t = warp + j * kDeltaWarps;
        float qq = 0.f, kk = 0.f;
#pragma unroll
        for (int n = 0; n < kDeltaPre; ++n) { qq = fmaf(pq[j][n], pq[j][n], qq); kk = fmaf(pk[j][n], pk[j][n], kk); }
        qq = a.q_scale / sqrtf(warp_sum(qq) + a.unit_eps);
        kk = 1.f / sqrtf(warp_sum(kk) + a.unit_eps);
        if (t < nt) {
#pragma unroll
          for (int n = 0; n < kDeltaPre; ++n) {
            const int i = lane + 32 * n;
            if (i < lanes * NS) {
              const int at = t * ldk + (i / NS) * kPad + i % NS;
              qs[at] = pq[j][n] * qq;
              ks[at] = pk[j][n] * kk;
            }
          }
        }
      }
    } else {
      for (int t = warp; t < nt; t += kDeltaWarps) {
        const float* xr = qkv + (size_t)(e.y + t0 + t) * a.ldx;
        float qq = 0.f, kk = 0.f;
        for (int i = lane; i < D; i += 32) {
          const float qv = xr[q_col + i], kv = xr[k_col + i];
          qq = fmaf(qv, qv, qq);
          kk = fmaf(kv, kv, kk);
        }
        qq = a.q_scale / sqrtf(warp_sum(qq) + a.unit_eps);
        kk = 1.f / sqrtf(warp_sum(kk) + a.unit_eps);
        for (int i = lane; i < lanes * NS; i += 32) {
          const int at = t * ldk + (i / NS) * kPad + i % NS;
          qs[at] = i < D ? xr[q_col + i] * qq : 0.f;
          ks[at] = i < D ? xr[k_col + i] * kk : 0.f;
        }
      }
    }
    for (int i = tid; i < nt * cpb; i += kDeltaWarps * 32) {
      const int t = i / cpb, c = i - t * cpb;
      vs[i] = (blockIdx.z * cpb + c < a.V) ? qkv[(size_t)(e.y + t0 + t) * a.ldx + v_col + c] : 0.f;
    }
    if (tid < nt) {
      const E* pr = proj + (size_t)(e.y + t0 + tid) * a.ldp;
      const float b = d_to_f(pr[a.b_off + h]), x = d_to_f(pr[a.a_off + h]) + dtb;
      const float sp = x > 20.f ? x : log1pf(expf(x));
      bg[4 * tid] = 1.f / (1.f + expf(-b));
      bg[4 * tid + 1] = neg_a * sp;
    }
    __syncthreads();
    if (pre && t0 + CB < e.z) fetch(t0 + CB);
    // ---- A and P of the pass (pairs s <= t), and the running sums of log g
    for (int idx = tid; idx < CB * CB; idx += kDeltaWarps * 32) {
      const int t = idx / CB, sx = idx - t * CB;
      if (t >= nt || sx > t) continue;
      float kkd = 0.f, qkd = 0.f;
      for (int pb = 0; pb < lanes; ++pb) {
#pragma unroll
        for (int n = 0; n < NS; n += 4) {
          const float4 kt = *reinterpret_cast<const float4*>(ks + t * ldk + pb * kPad + n);
          const float4 qt = *reinterpret_cast<const float4*>(qs + t * ldk + pb * kPad + n);
          const float4 kx = *reinterpret_cast<const float4*>(ks + sx * ldk + pb * kPad + n);
          kkd = fmaf(kt.x, kx.x, kkd); kkd = fmaf(kt.y, kx.y, kkd); kkd = fmaf(kt.z, kx.z, kkd); kkd = fmaf(kt.w, kx.w, kkd);
          qkd = fmaf(qt.x, kx.x, qkd); qkd = fmaf(qt.y, kx.y, qkd); qkd = fmaf(qt.z, kx.z, qkd); qkd = fmaf(qt.w, kx.w, qkd);
        }
      }
      float dsum = 0.f;
      for (int r = sx + 1; r <= t; ++r) dsum += bg[4 * r + 1];
      const float dec = expf(dsum);
      Am[idx] = bg[4 * t] * dec * kkd;
      Pm[idx] = dec * qkd;
      if (sx == 0) bg[4 * t + 2] = dsum + bg[1];   // running sum of log g through row t
    }
    __syncthreads();
    // ---- read-outs of the old state for all rows of the pass
    float wa[CB], za[CB];
#pragma unroll
    for (int t = 0; t < CB; ++t) {
      wa[t] = 0.f; za[t] = 0.f;
      if (t < nt) {
        const float4* kp = reinterpret_cast<const float4*>(ks + t * ldk + p * kPad);
        const float4* qp = reinterpret_cast<const float4*>(qs + t * ldk + p * kPad);
        float w2 = 0.f, z2 = 0.f;
#pragma unroll
        for (int n = 0; n < NS / 4; ++n) {
          const float4 kf = kp[n], qf = qp[n];
          wa[t] = fmaf(s[4 * n], kf.x, wa[t]); w2 = fmaf(s[4 * n + 1], kf.y, w2);
          wa[t] = fmaf(s[4 * n + 2], kf.z, wa[t]); w2 = fmaf(s[4 * n + 3], kf.w, w2);
          za[t] = fmaf(s[4 * n], qf.x, za[t]); z2 = fmaf(s[4 * n + 1], qf.y, z2);
          za[t] = fmaf(s[4 * n + 2], qf.z, za[t]); z2 = fmaf(s[4 * n + 3], qf.w, z2);
        }
        wa[t] += w2; za[t] += z2;
      }
    }
    for (int off = 1; off < lanes; off <<= 1) {
#pragma unroll
      for (int t = 0; t < CB; ++t) {
        wa[t] += __shfl_xor_sync(0xffffffffu, wa[t], off);
        za[t] += __shfl_xor_sync(0xffffffffu, za[t], off);
      }
    }
    // ---- the substitution for u and the outputs (every lane of a column does it: all of them need u)
    float u[CB];
    float* orow = o + (size_t)(e.y + t0) * (a.H * a.V) + h * a.V + c0;
#pragma unroll
    for (int t = 0; t < CB; ++t) {
      u[t] = 0.f;
      if (t < nt) {
        const float gam = expf(bg[4 * t + 2]);
        float ut = bg[4 * t] * (vs[t * cpb + cl] - gam * wa[t]);
        float ot = gam * za[t];
#pragma unroll
        for (int sx = 0; sx < t; ++sx) {
          ut = fmaf(-Am[t * CB + sx], u[sx], ut);
          ot = fmaf(Pm[t * CB + sx], u[sx], ot);
        }
        u[t] = ut;
        ot = fmaf(Pm[t * CB + t], ut, ot);
        if (p == 0 && c0 < a.V) orow[(size_t)t * (a.H * a.V)] = ot;
      }
    }
    // ---- the state after the pass
    const float c_last = bg[4 * (nt - 1) + 2];
    const float g_all = expf(c_last);
#pragma unroll
    for (int n = 0; n < NS; ++n) s[n] *= g_all;
#pragma unroll
    for (int t = 0; t < CB; ++t) {
      if (t < nt) {
        const float ud = u[t] * expf(c_last - bg[4 * t + 2]);
        const float4* kp = reinterpret_cast<const float4*>(ks + t * ldk + p * kPad);
#pragma unroll
        for (int n = 0; n < NS / 4; ++n) {
          const float4 kf = kp[n];
          s[4 * n] = fmaf(kf.x, ud, s[4 * n]); s[4 * n + 1] = fmaf(kf.y, ud, s[4 * n + 1]);
          s[4 * n + 2] = fmaf(kf.z, ud, s[4 * n + 2]); s[4 * n + 3] = fmaf(kf.w, ud, s[4 * n + 3]);
        }
      }
    }
  }
  if (c0 < a.V) {
    float* sp = St + (((size_t)e.x * a.H + h) * a.V + c0) * D + r0;
#pragma unroll
    for (int n = 0; n < NS; ++n)
      if (r0 + n < D) sp[n] = s[n];
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

template <typename E, int CPT, int NS>
static int launch_delta(const float* qkv, const void* proj, float* St, float* o, int n_ent, const DeltaRun& a,
                        cudaStream_t s) {
  const int cpb = delta_cols_per_cta(a.D, NS, CPT);
  const size_t smem = sizeof(float) * ((size_t)2 * kDeltaBlock * delta_lanes(a.D, NS) * delta_pad(NS) + kDeltaBlock * cpb + 3 * kDeltaBlock);
  const dim3 grid(n_ent, a.H, (a.V + cpb - 1) / cpb);
  DLI_LAUNCH("delta_rule", (delta_rule_kernel<E, CPT, NS>), grid, dim3(kDeltaWarps * 32), smem, s, qkv, (const E*)proj, St, o, a);
  return DLI_OK;
}

template <typename E>
static int launch_delta_block(const float* qkv, const void* proj, float* St, float* o, int n_ent, const DeltaRun& a,
                              cudaStream_t s) {
  const int lanes = delta_lanes(a.D, 16), cpb = delta_cols_per_cta(a.D, 16, 1);
  const size_t smem = sizeof(float) * ((size_t)2 * kDeltaBlock * (lanes * delta_pad(16) + 4) + kDeltaBlock * cpb + 4 * kDeltaBlock +
                                       2 * kDeltaBlock * kDeltaBlock);
  const dim3 grid(n_ent, a.H, (a.V + cpb - 1) / cpb);
  DLI_LAUNCH("delta_rule_block", delta_rule_block_kernel<E>, grid, dim3(kDeltaWarps * 32), smem, s, qkv, (const E*)proj, St, o, a);
  return DLI_OK;
}

template <typename E>
static int dispatch_delta(const float* qkv, const void* proj, float* St, float* o, int n_ent, const DeltaRun& a,
                          cudaStream_t s, int blocked) {
  if (blocked) return launch_delta_block<E>(qkv, proj, St, o, n_ent, a, s);
  // two columns per thread (the fewest instructions) where that still gives every SM a few CTAs; else one, and for
  // few rows of a small key size four state rows per lane, which spreads a decode row's state over 4x as many CTAs
  auto ctas = [&](int NS, int cpt) {
    const int cpb = delta_cols_per_cta(a.D, NS, cpt);
    return (long)n_ent * a.H * ((a.V + cpb - 1) / cpb);
  };
  const long sms = sm_count_cached();
  if (ctas(16, 2) >= 2 * sms) return launch_delta<E, 2, 16>(qkv, proj, St, o, n_ent, a, s);
  // fewer columns than that: eight (four) state rows per lane give a scheduler more warps to switch between, as long
  // as all CTAs are still resident at once (two per SM at these register counts)
  if (a.D > 128 || ctas(8, 1) > 2 * sms) return launch_delta<E, 1, 16>(qkv, proj, St, o, n_ent, a, s);
  if (ctas(4, 1) > 2 * sms) return launch_delta<E, 1, 8>(qkv, proj, St, o, n_ent, a, s);
  return launch_delta<E, 1, 4>(qkv, proj, St, o, n_ent, a, s);
}

}  // namespace dli

using namespace dli;

extern "C" {

int dli_delta_rule_ragged(const float* qkv, const void* proj, float* St, float* o, const int32_t* ent, int n_ent, int H,
                          int G, int D, int V, int ldx, int ldp, int b_off, int a_off, const float* a_log,
                          const float* dt_bias, float q_scale, float unit_eps, int blocked, int dt, dli_stream_t stream) {
  DLI_CHECK_ARG(qkv && proj && St && o && ent && a_log && dt_bias, "dli_delta_rule_ragged: null pointer");
  DLI_CHECK_ARG(H > 0 && G > 0 && H % G == 0 && D > 0 && D <= 512 && V > 0 && ldx >= 2 * G * D + H * V,
                "dli_delta_rule_ragged: H=%d G=%d D=%d V=%d ldx=%d (H %% G == 0, D <= 512)", H, G, D, V, ldx);
  DLI_CHECK_ARG((reinterpret_cast<uintptr_t>(ent) & 15u) == 0, "dli_delta_rule_ragged: ent must be 16-byte aligned");
  DLI_CHECK_ARG(dt == 0 || dt == 1, "element type %d: 0 = bf16, 1 = float", dt);
  if (n_ent <= 0) return DLI_OK;
  DeltaRun a{ent, H, G, D, V, ldx, ldp, b_off, a_off, a_log, dt_bias, q_scale, unit_eps};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return dt == 0 ? dispatch_delta<bf16>(qkv, proj, St, o, n_ent, a, s, blocked) : dispatch_delta<float>(qkv, proj, St, o, n_ent, a, s, blocked);
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
