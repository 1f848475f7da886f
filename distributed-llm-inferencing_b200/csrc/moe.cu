// Mixture-of-experts feed-forward for a RAGGED step: the router and the expert activation.
//
//   dli_moe_route   logits z = W_r h (fp32), scores s = softmax(z) over all router outputs; the `top` outputs with
//                   the largest s + correction are chosen; their weights are s / (sum of the chosen s + 1e-20), or,
//                   without renormalisation, s itself, in both cases times `wscale`.  With groups > 1 the outputs form
//                   that many equal groups of neighbours, a group's score is its largest s + correction, and only
//                   outputs of the `keep` best groups can be chosen.
//                   The last n_identity router outputs are experts that return their input: their weights are
//                   summed into idw[row].  Written: the dense weight row wts[row, 0 .. n_real) (0 for experts that
//                   were not chosen), idw[row], and the choice itself (sel_idx / sel_w [row, top]).
//   dli_moe_act     the experts' activation on the stacked gate/up projection of all experts:
//                   g = min(g, limit), u = clamp(u, -limit, limit), a = g * sigmoid(alpha g) * (u + 1), times the
//                   expert's routing weight, so that ONE down projection over the concatenated experts is the
//                   weighted sum of their outputs.  A shared expert (its own size and limit, weight 1) is the last
//                   block.  mode 1: experts without a gate, a = max(u, 0)^2 on the stacked up projections.
#include <math.h>

#include "common.cuh"
#include "moe_route.cuh"

namespace dli {

template <typename E> __device__ __forceinline__ float x_to_f(E v);
template <> __device__ __forceinline__ float x_to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float x_to_f<bf16>(bf16 v) { return __bfloat162float(v); }
template <typename E> __device__ __forceinline__ E x_from_f(float v);
template <> __device__ __forceinline__ float x_from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 x_from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

// One CTA per row: a warp per router output for the logits, then one warp does the softmax and the choice (moe_route.cuh).
__global__ void __launch_bounds__(512)
moe_route_kernel(const float* __restrict__ h, int d, RouteArgs ra) {
  extern __shared__ float zs[];  // [n_out] scores, [n_out] choice scores, [groups] group scores
  pdl_wait();
  pdl_trigger();
  moe_route_row(h + (size_t)blockIdx.x * d, d, blockIdx.x, ra, zs);
}

struct MoeAct {
  int n_exp, ff;            // routed experts and their size; columns [e*2*ff, +ff) gate, [e*2*ff + ff, +ff) up
  float limit;
  int ff_s;                 // shared expert's size (0: none), its gate/up follow the routed experts'
  float limit_s;
  float alpha;              // g * sigmoid(alpha * g)
  int ld;                   // row stride of gu
  int mode;                 // 0: clamped gated form; 1: no gate, max(u, 0)^2, columns [e*ff, +ff) of gu (shared: after them)
  int vec;                  // mode 1: sizes and pointers allow 16-byte accesses
};

// act[row, e*ff + f] and act[row, n_exp*ff + f] (shared); a row's channels go to one CTA, or to several for few rows.
template <typename E>
__global__ void __launch_bounds__(256)
moe_act_kernel(const E* __restrict__ gu, const float* __restrict__ wts, E* __restrict__ act, MoeAct a) {
  pdl_wait();
  pdl_trigger();
  const size_t row = blockIdx.x;
  const E* g = gu + row * a.ld;
  const int F = a.n_exp * a.ff + a.ff_s;
  E* out = act + row * F;
  if (a.mode == 1 && a.vec) {
    // experts without a gate, 16 bytes per thread and access: the V elements lie in one expert (ff, ff_s multiples of V)
    constexpr int V = 16 / (int)sizeof(E);
    for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * V; i < F; i += blockDim.x * gridDim.y * V) {
      const float wt = i < a.n_exp * a.ff ? wts[row * a.n_exp + i / a.ff] : 1.f;
      uint4 o = make_uint4(0, 0, 0, 0);
      if (wt != 0.f) {
        const uint4 u = *reinterpret_cast<const uint4*>(g + i);
        if constexpr (sizeof(E) == 2) {
          float f[8];
          unpack8(u, f);
#pragma unroll
          for (int k = 0; k < 8; ++k) { const float r = fmaxf(f[k], 0.f); f[k] = r * r * wt; }
          o = pack8(f);
        } else {
          const float f[4] = {__uint_as_float(u.x), __uint_as_float(u.y), __uint_as_float(u.z), __uint_as_float(u.w)};
          float r[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) { const float t = fmaxf(f[k], 0.f); r[k] = t * t * wt; }
          o = make_uint4(__float_as_uint(r[0]), __float_as_uint(r[1]), __float_as_uint(r[2]), __float_as_uint(r[3]));
        }
      }
      *reinterpret_cast<uint4*>(out + i) = o;
    }
    return;
  }
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < F; i += blockDim.x * gridDim.y) {
    float gv, uv, lim, wt;
    if (a.mode == 1) {
      wt = 1.f;
      if (i < a.n_exp * a.ff) {
        wt = wts[row * a.n_exp + i / a.ff];
        if (wt == 0.f) { out[i] = x_from_f<E>(0.f); continue; }
      }
      const float u = fmaxf(x_to_f(g[i]), 0.f);
      out[i] = x_from_f<E>(u * u * wt);
      continue;
    }
    if (i < a.n_exp * a.ff) {
      const int e = i / a.ff, f = i - e * a.ff;
      wt = wts[row * a.n_exp + e];
      if (wt == 0.f) { out[i] = x_from_f<E>(0.f); continue; }
      gv = x_to_f(g[(size_t)e * 2 * a.ff + f]);
      uv = x_to_f(g[(size_t)e * 2 * a.ff + a.ff + f]);
      lim = a.limit;
    } else {
      const int f = i - a.n_exp * a.ff;
      wt = 1.f;
      gv = x_to_f(g[(size_t)a.n_exp * 2 * a.ff + f]);
      uv = x_to_f(g[(size_t)a.n_exp * 2 * a.ff + a.ff_s + f]);
      lim = a.limit_s;
    }
    gv = fminf(gv, lim);
    uv = fminf(fmaxf(uv, -lim), lim);
    const float y = gv / (1.f + expf(-a.alpha * gv)) * (uv + 1.f);
    out[i] = x_from_f<E>(y * wt);
  }
}


// ---- few rows (decode): only the chosen experts' weights are read ------------------------------------------------
// dli_moe_sel_act: for row r and its k-th choice e = sel_idx[r, k] (k == top: the shared expert) the gate and up
// rows of that expert are streamed (one warp per output, 16-byte loads) and the weighted activation goes to the
// compact act_sel [rows, top*ff + ff_s] (zeros for a pass-through choice).  dli_moe_sel_down: y[r, c] = sum over the
// choices of act_sel[r, k, :] . w_down[c, e_k*ff : +ff] plus the shared block.
__device__ __forceinline__ float dot8(const uint4& w, const float* x) {
  float f[8];
  unpack8(w, f);
  float a = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) a = fmaf(f[j], x[j], a);
  return a;
}

constexpr int kSelWarps = 8;
constexpr int kSelPerWarp = 4;  // activation outputs per warp (the down projection: one output per warp)

__global__ void __launch_bounds__(kSelWarps * 32)
moe_sel_act_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w_gu, const int32_t* __restrict__ sel_idx,
                   const float* __restrict__ sel_w, bf16* __restrict__ act_sel, int d, int top, MoeAct a) {
  extern __shared__ float xs[];  // [d]
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x, k = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool shared = k == top;
  const int ff = shared ? a.ff_s : a.ff;
  const int f0 = (blockIdx.z * kSelWarps + warp) * kSelPerWarp;
  if (blockIdx.z * kSelWarps * kSelPerWarp >= ff) return;
  bf16* out = act_sel + (size_t)row * (top * a.ff + a.ff_s) + (shared ? top * a.ff : k * a.ff);
  const int e = shared ? a.n_exp : sel_idx[row * top + k];
  if (!shared && e >= a.n_exp) {  // a pass-through choice: nothing to stream
    for (int f = f0 + lane; f < min(f0 + kSelPerWarp, ff); f += 32) out[f] = __float2bfloat16_rn(0.f);
    return;
  }
  for (int c = threadIdx.x; c < d; c += blockDim.x) xs[c] = __bfloat162float(x[(size_t)row * d + c]);
  __syncthreads();
  const float wt = shared ? 1.f : sel_w[row * top + k];
  const float lim = shared ? a.limit_s : a.limit;
  if (a.mode == 1) {
    // experts without a gate: one weight row per output, two outputs at a time
    const bf16* base1 = w_gu + (size_t)e * a.ff * d;
    for (int f = f0; f < min(f0 + kSelPerWarp, ff); f += 2) {
      const int f1 = min(f + 1, ff - 1);
      const bf16* r0 = base1 + (size_t)f * d;
      const bf16* r1 = base1 + (size_t)f1 * d;
      float u0 = 0.f, u1 = 0.f;
      int c = lane * 8;
      for (; c + 768 < d; c += 1024) {  // eight 16-byte loads in flight per lane
        uint4 w0[4], w1[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) { w0[i] = ld_stream_16B(r0 + c + i * 256); w1[i] = ld_stream_16B(r1 + c + i * 256); }
#pragma unroll
        for (int i = 0; i < 4; ++i) { u0 += dot8(w0[i], xs + c + i * 256); u1 += dot8(w1[i], xs + c + i * 256); }
      }
      for (; c < d; c += 256) {
        u0 += dot8(ld_stream_16B(r0 + c), xs + c);
        u1 += dot8(ld_stream_16B(r1 + c), xs + c);
      }
      u0 = warp_sum(u0); u1 = warp_sum(u1);
      if (lane < 2 && f + lane < ff) {
        float u = lane ? u1 : u0;
        u = fmaxf(__bfloat162float(__float2bfloat16_rn(u)), 0.f);  // the projection's output is a bf16 row, as on the dense path
        out[f + lane] = __float2bfloat16_rn(u * u * wt);
      }
    }
    return;
  }
  const bf16* base = w_gu + (size_t)e * 2 * a.ff * d;  // the shared expert's block follows the n_exp routed ones
  for (int f = f0; f < min(f0 + kSelPerWarp, ff); f += 2) {
    // two outputs at a time: the gate and up rows of both are streamed together (eight 16-byte loads in flight per lane)
    const int f1 = min(f + 1, ff - 1);
    const bf16* gr0 = base + (size_t)f * d;
    const bf16* ur0 = base + (size_t)(ff + f) * d;
    const bf16* gr1 = base + (size_t)f1 * d;
    const bf16* ur1 = base + (size_t)(ff + f1) * d;
    float g0 = 0.f, u0 = 0.f, g1 = 0.f, u1 = 0.f;
    int c = lane * 8;
#pragma unroll 2
    for (; c + 256 < d; c += 512) {
      const uint4 a0 = ld_stream_16B(gr0 + c), b0 = ld_stream_16B(ur0 + c), a1 = ld_stream_16B(gr1 + c), b1 = ld_stream_16B(ur1 + c);
      const uint4 a2 = ld_stream_16B(gr0 + c + 256), b2 = ld_stream_16B(ur0 + c + 256), a3 = ld_stream_16B(gr1 + c + 256),
                  b3 = ld_stream_16B(ur1 + c + 256);
      g0 += dot8(a0, xs + c) + dot8(a2, xs + c + 256);
      u0 += dot8(b0, xs + c) + dot8(b2, xs + c + 256);
      g1 += dot8(a1, xs + c) + dot8(a3, xs + c + 256);
      u1 += dot8(b1, xs + c) + dot8(b3, xs + c + 256);
    }
    for (; c < d; c += 256) {
      g0 += dot8(ld_stream_16B(gr0 + c), xs + c);
      u0 += dot8(ld_stream_16B(ur0 + c), xs + c);
      g1 += dot8(ld_stream_16B(gr1 + c), xs + c);
      u1 += dot8(ld_stream_16B(ur1 + c), xs + c);
    }
    g0 = warp_sum(g0); u0 = warp_sum(u0); g1 = warp_sum(g1); u1 = warp_sum(u1);
    if (lane < 2 && f + lane < ff) {
      float g = lane ? g1 : g0, u = lane ? u1 : u0;
      g = __bfloat162float(__float2bfloat16_rn(g));  // the projection's output is a bf16 row, as on the dense path
      u = __bfloat162float(__float2bfloat16_rn(u));
      g = fminf(g, lim);
      u = fminf(fmaxf(u, -lim), lim);
      out[f + lane] = __float2bfloat16_rn(g / (1.f + expf(-a.alpha * g)) * (u + 1.f) * wt);
    }
  }
}

__global__ void __launch_bounds__(kSelWarps * 32)
moe_sel_down_kernel(const bf16* __restrict__ act_sel, const bf16* __restrict__ w_down, const int32_t* __restrict__ sel_idx,
                    bf16* __restrict__ y, int d, int top, MoeAct a) {
  extern __shared__ float as[];  // [top*ff + ff_s]
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_sel = top * a.ff + a.ff_s, F = a.n_exp * a.ff + a.ff_s;
  for (int i = threadIdx.x; i < n_sel; i += blockDim.x) as[i] = __bfloat162float(act_sel[(size_t)row * n_sel + i]);
  __syncthreads();
  const int c = blockIdx.y * kSelWarps + warp;  // one output per warp
  if (c >= d) return;
  const bf16* wr = w_down + (size_t)c * F;
  float acc = 0.f;
  for (int k = 0; k <= top; ++k) {
    const bool shared = k == top;
    const int e = shared ? a.n_exp : sel_idx[row * top + k];
    if (!shared && e >= a.n_exp) continue;
    const int ff = shared ? a.ff_s : a.ff;
    const bf16* seg = wr + (size_t)e * a.ff;  // the shared block starts at n_exp * ff
    const float* av = as + (shared ? top * a.ff : k * a.ff);
    int f = lane * 8;
    for (; f + 7 * 256 < ff; f += 8 * 256) {  // eight 16-byte loads in flight per lane
      uint4 w[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) w[i] = ld_stream_16B(seg + f + i * 256);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc += dot8(w[i], av + f + i * 256);
    }
    for (; f + 3 * 256 < ff; f += 4 * 256) {
      const uint4 w0 = ld_stream_16B(seg + f), w1 = ld_stream_16B(seg + f + 256), w2 = ld_stream_16B(seg + f + 512),
                  w3 = ld_stream_16B(seg + f + 768);
      acc += dot8(w0, av + f) + dot8(w1, av + f + 256) + dot8(w2, av + f + 512) + dot8(w3, av + f + 768);
    }
    for (; f < ff; f += 256) acc += dot8(ld_stream_16B(seg + f), av + f);
  }
  acc = warp_sum(acc);
  if (lane == 0) y[(size_t)row * d + c] = __float2bfloat16_rn(acc);
}

}  // namespace dli

using namespace dli;

extern "C" {

int dli_moe_route(const float* h, const float* w_router, const float* correction, float* wts, float* idw, int32_t* sel_idx,
                  float* sel_w, int rows, int d, int n_out, int n_real, int top, int groups, int keep, float wscale,
                  int renorm, dli_stream_t stream) {
  DLI_CHECK_ARG(h && w_router && wts && idw && sel_idx && sel_w, "dli_moe_route: null pointer");
  if (groups < 1) groups = 1;
  DLI_CHECK_ARG(groups == 1 || (n_out % groups == 0 && keep >= 1 && keep <= groups && keep * (n_out / groups) >= top),
                "dli_moe_route: %d router outputs in %d groups of which %d are kept, top %d", n_out, groups, keep, top);
  DLI_CHECK_ARG(d > 0 && n_out > 0 && n_real >= 0 && n_real <= n_out && top > 0 && top <= n_out && n_out <= 4096,
                "dli_moe_route: %d router outputs (%d real experts), top %d", n_out, n_real, top);
  if (rows <= 0) return DLI_OK;
  RouteArgs ra{w_router, correction, wts, idw, sel_idx, sel_w, n_out, n_real, top, groups, keep, wscale, renorm};
  DLI_LAUNCH("moe_route", moe_route_kernel, dim3(rows), dim3(rows <= 64 ? 512 : 256), (size_t)(2 * n_out + groups) * sizeof(float),
             static_cast<cudaStream_t>(stream), h, d, ra);
  return DLI_OK;
}

int dli_moe_act(const void* gu, const float* wts, void* act, int rows, int n_exp, int ff, float limit, int ff_s,
                float limit_s, float alpha, int ld, int dt, int mode, dli_stream_t stream) {
  DLI_CHECK_ARG(gu && act && (wts || n_exp == 0) && n_exp >= 0 && ff >= 0 && ff_s >= 0 && n_exp * ff + ff_s > 0 &&
                    (mode == 0 || mode == 1) && ld >= (mode == 1 ? 1 : 2) * (n_exp * ff + ff_s),
                "dli_moe_act: null pointer or bad shape");
  DLI_CHECK_ARG(dt == 0 || dt == 1, "element type %d: 0 = bf16, 1 = float", dt);
  if (rows <= 0) return DLI_OK;
  const int per = dt == 0 ? 8 : 4;
  const int vec = mode == 1 && ff % per == 0 && ff_s % per == 0 && ld % per == 0 && aligned16(gu) && aligned16(act);
  MoeAct a{n_exp, ff, limit, ff_s, limit_s, alpha, ld, mode, vec};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int work = (n_exp * ff + ff_s) / (vec ? per : 1);
  const int gy = rows <= 64 ? min(64, (work + 255) / 256) : (work >= 4096 ? 4 : 1);  // few rows, or long rows: several CTAs per row
  if (dt == 0) DLI_LAUNCH("moe_act", moe_act_kernel<bf16>, dim3(rows, gy), dim3(256), 0, s, (const bf16*)gu, wts, (bf16*)act, a);
  else DLI_LAUNCH("moe_act", moe_act_kernel<float>, dim3(rows, gy), dim3(256), 0, s, (const float*)gu, wts, (float*)act, a);
  return DLI_OK;
}

int dli_moe_sel_supported(int d, int ff, int ff_s, int top) {
  return d % 8 == 0 && ff % 8 == 0 && ff_s % 8 == 0 && (size_t)d * 4 <= 96 * 1024 && ((size_t)top * ff + ff_s) * 4 <= 96 * 1024;
}

int dli_moe_sel_bf16(const void* x, const void* w_gu, const void* w_down, const int32_t* sel_idx, const float* sel_w,
                     void* act_sel, void* y, int rows, int d, int n_exp, int top, int ff, float limit, int ff_s,
                     float limit_s, float alpha, int mode, dli_stream_t stream) {
  DLI_CHECK_ARG(x && w_gu && w_down && sel_idx && sel_w && act_sel && y && (mode == 0 || mode == 1), "dli_moe_sel_bf16: null pointer");
  DLI_CHECK_ARG(n_exp >= 0 && top >= 0 && dli_moe_sel_supported(d, ff, ff_s, top) && aligned16(w_gu) && aligned16(w_down),
                "dli_moe_sel_bf16: sizes d=%d ff=%d ff_s=%d must be multiples of 8 and fit shared memory", d, ff, ff_s);
  if (rows <= 0) return DLI_OK;
  MoeAct a{n_exp, ff, limit, ff_s, limit_s, alpha, 0, mode, 0};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  static PerDeviceOnce once_a, once_d;
  DLI_ONCE_PER_DEVICE(once_a, dev, DLI_CUDA_CALL(cudaFuncSetAttribute(moe_sel_act_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024)));
  DLI_ONCE_PER_DEVICE(once_d, dev2, DLI_CUDA_CALL(cudaFuncSetAttribute(moe_sel_down_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024)));
  const int per = kSelWarps * kSelPerWarp;
  const int ffm = ff > ff_s ? ff : ff_s;
  DLI_LAUNCH("moe_sel_act", moe_sel_act_kernel, dim3(rows, top + (ff_s ? 1 : 0), (ffm + per - 1) / per), dim3(kSelWarps * 32),
             (size_t)d * 4, s, (const bf16*)x, (const bf16*)w_gu, sel_idx, sel_w, (bf16*)act_sel, d, top, a);
  DLI_LAUNCH("moe_sel_down", moe_sel_down_kernel, dim3(rows, (d + kSelWarps - 1) / kSelWarps), dim3(kSelWarps * 32),
             ((size_t)top * ff + ff_s) * 4, s, (const bf16*)act_sel, (const bf16*)w_down, sel_idx, (bf16*)y, d, top, a);
  return DLI_OK;
}

}  // extern "C"
