// The router of a mixture of experts for ONE row, shared by dli_moe_route and by kernels that have the router's input row at
// hand (the closing kernel of pre-norm layers).  Every thread of the CTA calls it; zs is shared scratch of
// 2 * n_out + groups floats.  Logits in fp32, a warp per router output; then one warp does the softmax, the groups and
// the choice.  Nothing after the call may need all threads: the warps other than the first return early.
#pragma once
#include <math.h>

#include "common.cuh"

namespace dli {

struct RouteArgs {
  const float* wr;        // [n_out, d] fp32
  const float* corr;      // [n_out] or NULL: added to the scores for the choice only
  float* wts;             // [rows, n_real]: weight per real expert, 0 = not chosen
  float* idw;             // [rows]: summed weight of the chosen pass-through outputs
  int32_t* sel_idx;       // [rows, top]
  float* sel_w;           // [rows, top]
  int n_out, n_real, top;
  int groups, keep;       // groups > 1: only outputs of the `keep` best of that many equal groups can be chosen
  float wscale;
  int renorm;             // 1: weights divided by the sum of the chosen scores
};

// hr may have been written earlier in the same kernel (no __restrict__: plain coherent loads).
__device__ __forceinline__ void moe_route_row(const float* hr, int d, size_t row, const RouteArgs& ra, float* zs) {
  const float* __restrict__ wr = ra.wr;
  const float* __restrict__ corr = ra.corr;
  float* __restrict__ wts = ra.wts;
  float* __restrict__ idw = ra.idw;
  int32_t* __restrict__ sel_idx = ra.sel_idx;
  float* __restrict__ sel_w = ra.sel_w;
  const int n_out = ra.n_out, n_real = ra.n_real, top = ra.top, groups = ra.groups, keep = ra.keep, renorm = ra.renorm;
  const float wscale = ra.wscale;
  float* cs = zs + n_out;
  float* gm = cs + n_out;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int o = warp; o < n_out; o += nw) {
    const float* w = wr + (size_t)o * d;
    float acc = 0.f;
    if ((d & 3) == 0) {  // 16-byte loads, four in flight per lane
      const float4* h4 = reinterpret_cast<const float4*>(hr);
      const float4* w4 = reinterpret_cast<const float4*>(w);
#pragma unroll 4
      for (int c = lane; c < d / 4; c += 32) {
        const float4 a = h4[c], b = w4[c];
        acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc); acc = fmaf(a.z, b.z, acc); acc = fmaf(a.w, b.w, acc);
      }
    } else {
      for (int c = lane; c < d; c += 32) acc = fmaf(hr[c], w[c], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) zs[o] = acc;
  }
  __syncthreads();
  if (warp != 0) return;
  float mx = -INFINITY;
  for (int o = lane; o < n_out; o += 32) mx = fmaxf(mx, zs[o]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int o = lane; o < n_out; o += 32) sum += expf(zs[o] - mx);
  sum = warp_sum(sum);
  for (int o = lane; o < n_out; o += 32) {
    const float s = expf(zs[o] - mx) / sum;
    zs[o] = s;
    cs[o] = s + (corr ? corr[o] : 0.f);
    if (o < n_real) wts[row * n_real + o] = 0.f;
  }
  __syncwarp();
  if (groups > 1) {
    // a group's score is its largest choice score; the groups that are not among the `keep` best leave the choice
    const int per = n_out / groups;
    for (int g = lane; g < groups; g += 32) {
      float b = -INFINITY;
      for (int o = g * per; o < (g + 1) * per; ++o) b = fmaxf(b, cs[o]);
      gm[g] = b;
    }
    __syncwarp();
    for (int k = 0; k < keep; ++k) {
      float best = -INFINITY;
      int bi = 0x7fffffff;
      for (int g = lane; g < groups; g += 32) {
        const float c = gm[g];
        if (c > best && c != INFINITY) { best = c; bi = g; }
      }
      for (int off = 16; off > 0; off >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, off);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      if (lane == 0 && bi < groups) gm[bi] = INFINITY;  // kept
      __syncwarp();
    }
    for (int o = lane; o < n_out; o += 32)
      if (gm[o / per] != INFINITY) cs[o] = -INFINITY;
    __syncwarp();
  }
  // the `top` largest choice scores, one at a time (lowest index wins a tie)
  float chosen_sum = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int o = lane; o < n_out; o += 32) {
      const float c = cs[o];
      if (c > best) { best = c; bi = o; }
    }
    for (int off = 16; off > 0; off >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, off);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (bi >= n_out) bi = 0;  // fewer candidates than `top` (every score -inf or NaN): stay inside the row
    if (lane == 0) {
      cs[bi] = -INFINITY;
      sel_idx[row * top + k] = bi;
    }
    chosen_sum += zs[bi];
    __syncwarp();
  }
  const float inv = (renorm ? 1.f / (chosen_sum + 1e-20f) : 1.f) * wscale;
  if (lane == 0) {
    float ident = 0.f;
    for (int k = 0; k < top; ++k) {
      const int o = sel_idx[row * top + k];
      const float w = zs[o] * inv;
      sel_w[row * top + k] = w;
      if (o < n_real) wts[row * n_real + o] = w;
      else ident += w;
    }
    idw[row] = ident;
  }
}

}  // namespace dli
