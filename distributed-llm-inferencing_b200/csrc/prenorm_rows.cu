// Row-wise pieces of PRE-NORM layers on a ragged step (fp32 residual stream):
//
//   x <- x + ls * sublayer(norm(x) * w)        a weight vector per norm, a LAYER SCALE vector ls on the sublayer's result
//   the mixer reads its normed input through a TOKEN SHIFT: h_t + (h_(t-1) - h_t) * s, h_(t-1) the previous position's
//   normed row (zeros at position 0), kept per sequence slot between steps
//   after the layer a DEPTH AVERAGE: with X_0 the embedding output and X_(j+1) layer j's result, the stream handed on is
//   sum_j a[j] X_j over all results so far
//
// dli_layer_close does everything between two projections in one pass over the row: the scaled residual add (with an
// optional bias on the sublayer's result and the share of pass-through experts), the depth average, and the NEXT
// norm (fp32 and / or element-type output).  For steps of one row per entry (decode) it also applies the next mixer's
// token shift and advances the slot's previous row; where the norm feeds a mixture of experts it also runs the ROUTER on
// the normed row it has just written.  dli_token_shift_ragged is the shift for steps with portions of prompts, on the
// normed rows.
#include "common.cuh"
#include "moe_route.cuh"

namespace dli {

template <typename E> __device__ __forceinline__ float pn_to_f(E v);
template <> __device__ __forceinline__ float pn_to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float pn_to_f<bf16>(bf16 v) { return __bfloat162float(v); }
template <typename E> __device__ __forceinline__ E pn_from_f(float v);
template <> __device__ __forceinline__ float pn_from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 pn_from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float pn_block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}

struct LayerClose {
  const float* bias;      // [d] or NULL: added to the sublayer's result y
  const float* idw;       // [rows] or NULL: weight of the experts that pass their input through ...
  const float* h_in;      // ... and that input [rows, d]
  const float* ls;        // [d] or NULL: layer scale on (y + bias + idw * h_in)
  float* xs;              // stored results X_0, X_1, ..: X_j at xs + j * xs_stride
  size_t xs_stride;
  int n_prev;             // X_0 .. X_(n_prev - 1) are stored; this call stores X_(n_prev)
  const float* dwa;       // [n_prev + 1] or NULL: x <- sum_j dwa[j] X_j
  const float* w_next;    // [d] or NULL: weights of the norm that follows
  const float* shift;     // [d] or NULL: token shift of the normed row (one row per entry only)
  float* tail;            // [slots, d]: the previous position's normed row
  const int32_t* ent;
  float* out_f;           // [rows, d] or NULL
  float eps;
  int d;
  int has_route;          // the router of the feed-forward that follows runs on out_f's row
  RouteArgs route;
};

// VEC consecutive channels per thread and load: 16-byte loads of the fp32 rows (8 bytes of bf16) when the width allows
template <int VEC> __device__ __forceinline__ void ld_f(const float* p, float (&v)[VEC]);
template <> __device__ __forceinline__ void ld_f<1>(const float* p, float (&v)[1]) { v[0] = *p; }
template <> __device__ __forceinline__ void ld_f<4>(const float* p, float (&v)[4]) {
  const float4 u = *reinterpret_cast<const float4*>(p);
  v[0] = u.x; v[1] = u.y; v[2] = u.z; v[3] = u.w;
}
template <int VEC> __device__ __forceinline__ void st_f(float* p, const float (&v)[VEC]);
template <> __device__ __forceinline__ void st_f<1>(float* p, const float (&v)[1]) { *p = v[0]; }
template <> __device__ __forceinline__ void st_f<4>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <int VEC> __device__ __forceinline__ void ld_e(const float* p, float (&v)[VEC]) { ld_f<VEC>(p, v); }
template <int VEC> __device__ __forceinline__ void st_e(float* p, const float (&v)[VEC]) { st_f<VEC>(p, v); }
template <int VEC> __device__ __forceinline__ void ld_e(const bf16* p, float (&v)[VEC]);
template <> __device__ __forceinline__ void ld_e<1>(const bf16* p, float (&v)[1]) { v[0] = __bfloat162float(*p); }
template <> __device__ __forceinline__ void ld_e<4>(const bf16* p, float (&v)[4]) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  v[0] = bf_lo(u.x); v[1] = bf_hi(u.x); v[2] = bf_lo(u.y); v[3] = bf_hi(u.y);
}
template <int VEC> __device__ __forceinline__ void st_e(bf16* p, const float (&v)[VEC]);
template <> __device__ __forceinline__ void st_e<1>(bf16* p, const float (&v)[1]) { *p = __float2bfloat16_rn(v[0]); }
template <> __device__ __forceinline__ void st_e<4>(bf16* p, const float (&v)[4]) {
  *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]));
}

// One CTA per row.  Pass 1 forms the new x (and its sum of squares), pass 2 the next norm from the rows just written.
template <typename E, int VEC>
__global__ void __launch_bounds__(1024)
layer_close_kernel(const E* __restrict__ y, float* __restrict__ x, E* __restrict__ out_e, LayerClose a) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x, d = a.d;
  const size_t o = (size_t)row * d;
  const float iw = a.idw ? a.idw[row] : 0.f;
  float ss = 0.f;
  for (int c = threadIdx.x * VEC; c < d; c += blockDim.x * VEC) {
    float v[VEC];
    ld_f<VEC>(x + o + c, v);
    if (y) {
      float t[VEC];
      ld_e<VEC>(y + o + c, t);
      if (a.bias) {
        float b[VEC];
        ld_f<VEC>(a.bias + c, b);
#pragma unroll
        for (int i = 0; i < VEC; ++i) t[i] += b[i];
      }
      if (a.idw) {
        float h[VEC];
        ld_f<VEC>(a.h_in + o + c, h);
#pragma unroll
        for (int i = 0; i < VEC; ++i) t[i] = fmaf(iw, h[i], t[i]);
      }
      if (a.ls) {
        float l[VEC];
        ld_f<VEC>(a.ls + c, l);
#pragma unroll
        for (int i = 0; i < VEC; ++i) v[i] = fmaf(l[i], t[i], v[i]);
      } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) v[i] += t[i];
      }
    }
    if (a.dwa) {
      st_f<VEC>(a.xs + (size_t)a.n_prev * a.xs_stride + o + c, v);
      float u[VEC];
#pragma unroll
      for (int i = 0; i < VEC; ++i) u[i] = 0.f;
#pragma unroll 4
      for (int j = 0; j < a.n_prev; ++j) {  // the earlier results' loads do not depend on one another
        float p[VEC];
        ld_f<VEC>(a.xs + (size_t)j * a.xs_stride + o + c, p);
        const float w = a.dwa[j];
#pragma unroll
        for (int i = 0; i < VEC; ++i) u[i] = fmaf(w, p[i], u[i]);
      }
      const float w = a.dwa[a.n_prev];
#pragma unroll
      for (int i = 0; i < VEC; ++i) v[i] = fmaf(w, v[i], u[i]);
    }
    if (y || a.dwa) st_f<VEC>(x + o + c, v);
#pragma unroll
    for (int i = 0; i < VEC; ++i) ss = fmaf(v[i], v[i], ss);
  }
  if (!a.w_next) return;
  ss = pn_block_sum(ss, red);  // its barriers also order the writes of x above before the reads below
  const float r = 1.f / sqrtf(ss / d + a.eps);
  int slot = 0, pos = 0;
  if (a.shift) {
    const int4 e = reinterpret_cast<const int4*>(a.ent)[row];  // slot, first row (== row), 1, position
    slot = e.x; pos = e.w;
  }
  for (int c = threadIdx.x * VEC; c < d; c += blockDim.x * VEC) {
    float h[VEC], w[VEC];
    ld_f<VEC>(x + o + c, h);
    ld_f<VEC>(a.w_next + c, w);
#pragma unroll
    for (int i = 0; i < VEC; ++i) h[i] = h[i] * r * w[i];
    if (a.shift) {
      float* t = a.tail + (size_t)slot * d + c;
      float prev[VEC], s[VEC];
      ld_f<VEC>(t, prev);
      ld_f<VEC>(a.shift + c, s);
      st_f<VEC>(t, h);
#pragma unroll
      for (int i = 0; i < VEC; ++i) h[i] = fmaf((pos > 0 ? prev[i] : 0.f) - h[i], s[i], h[i]);
    }
    if (a.out_f) st_f<VEC>(a.out_f + o + c, h);
    if (out_e) st_e<VEC>(out_e + o + c, h);
  }
  if (a.has_route) {
    extern __shared__ float route_scratch[];  // 2 * n_out + groups floats
    __syncthreads();                          // the row of out_f is complete
    moe_route_row(a.out_f + o, d, row, a.route, route_scratch);
  }
}

// out[row] = h[row] + (prev - h[row]) * s with prev the previous row of the same entry, or, for an entry's first row, the
// slot's stored row (zeros at position 0).  The CTA of an entry's first row is the only one that touches the slot: it
// reads the stored row and then stores the entry's last row, channel by channel in the same thread.
template <typename E>
__global__ void __launch_bounds__(256)
token_shift_ragged_kernel(const float* __restrict__ h, const float* __restrict__ s, float* __restrict__ tail,
                          const int32_t* __restrict__ row_ent, const int32_t* __restrict__ ent, E* __restrict__ out, int d) {
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x;
  const int4 e = reinterpret_cast<const int4*>(ent)[row_ent[row]];  // slot, first row, rows, first position
  const bool first = row == e.y;
  const size_t o = (size_t)row * d;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < d; c += blockDim.x * gridDim.y) {
    const float cur = h[o + c];
    float prev;
    if (first) {
      float* t = tail + (size_t)e.x * d + c;
      prev = e.w > 0 ? *t : 0.f;
      *t = h[(size_t)(e.y + e.z - 1) * d + c];
    } else {
      prev = h[o - d + c];
    }
    out[o + c] = pn_from_f<E>(fmaf(prev - cur, s[c], cur));
  }
}

}  // namespace dli

using namespace dli;

extern "C" {

int dli_layer_close(const void* y, const float* bias, const float* idw, const float* h_in, const float* ls, float* x,
                    float* xs, size_t xs_stride, int n_prev, const float* dwa, const float* w_next, const float* shift,
                    float* tail, const int32_t* ent, float* out_f, void* out_e, int rows, int d, float eps, int dt,
                    const float* w_router, const float* correction, float* r_wts, float* r_idw, int32_t* r_sel_idx,
                    float* r_sel_w, int n_out, int n_real, int top, int groups, int keep, float wscale, int renorm,
                    dli_stream_t stream) {
  DLI_CHECK_ARG(x && d > 0, "dli_layer_close: null pointer or empty shape");
  DLI_CHECK_ARG(y || !(bias || idw || ls), "dli_layer_close: bias, pass-through share and layer scale need a sublayer result");
  DLI_CHECK_ARG(!idw || h_in, "dli_layer_close: the pass-through share needs its input rows");
  DLI_CHECK_ARG(!dwa || (xs && n_prev >= 0 && xs_stride >= (size_t)rows * d), "dli_layer_close: the depth average needs the stored results");
  DLI_CHECK_ARG(w_next || !(out_f || out_e || shift), "dli_layer_close: outputs need the norm's weights");
  DLI_CHECK_ARG(!w_next || out_f || out_e, "dli_layer_close: the norm has no output");
  DLI_CHECK_ARG(!shift || (tail && ent && (reinterpret_cast<uintptr_t>(ent) & 15u) == 0),
                "dli_layer_close: the token shift needs the slots' rows and a 16-byte aligned ent");
  DLI_CHECK_ARG(dt == 0 || dt == 1, "element type %d: 0 = bf16, 1 = float", dt);
  if (groups < 1) groups = 1;
  DLI_CHECK_ARG(!w_router || (out_f && !shift && r_wts && r_idw && r_sel_idx && r_sel_w && n_out > 0 && n_out <= 4096 &&
                              n_real >= 0 && n_real <= n_out && top > 0 && top <= n_out &&
                              (groups == 1 || (n_out % groups == 0 && keep >= 1 && keep <= groups && keep * (n_out / groups) >= top))),
                "dli_layer_close: the router needs the fp32 normed rows (no shift) and its outputs; %d outputs (%d real), top %d, "
                "%d groups of which %d are kept", n_out, n_real, top, groups, keep);
  if (rows <= 0) return DLI_OK;
  LayerClose a{bias, idw, h_in, ls, xs, xs_stride, n_prev, dwa, w_next, shift, tail, ent, out_f, eps, d, w_router ? 1 : 0,
               RouteArgs{w_router, correction, r_wts, r_idw, r_sel_idx, r_sel_w, n_out, n_real, top, groups, keep, wscale, renorm}};
  const size_t smem = w_router ? (size_t)(2 * n_out + groups) * sizeof(float) : 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // 16-byte accesses when every row and vector starts on such a boundary
  auto al = [](const void* p, uintptr_t n) { return (reinterpret_cast<uintptr_t>(p) & (n - 1)) == 0; };
  const bool vec = d % 4 == 0 && al(x, 16) && al(y, dt == 0 ? 8 : 16) && al(bias, 16) && al(h_in, 16) && al(ls, 16) && al(xs, 16) &&
                   xs_stride % 4 == 0 && al(w_next, 16) && al(shift, 16) && al(tail, 16) && al(out_f, 16) &&
                   al(out_e, dt == 0 ? 8 : 16);
  const int per = vec ? 4 : 1;
  int th = (rows <= 64 && d >= 2048 * per) ? 1024 : (d >= 256 * per ? 256 : 128);
  if (w_router && th < (rows <= 64 ? 512 : 256)) th = rows <= 64 ? 512 : 256;  // a warp per router output; few rows: more warps for the logits
  if (dt == 0) {
    if (vec) DLI_LAUNCH("layer_close", (layer_close_kernel<bf16, 4>), dim3(rows), dim3(th), smem, s, (const bf16*)y, x, (bf16*)out_e, a);
    else DLI_LAUNCH("layer_close", (layer_close_kernel<bf16, 1>), dim3(rows), dim3(th), smem, s, (const bf16*)y, x, (bf16*)out_e, a);
  } else {
    if (vec) DLI_LAUNCH("layer_close", (layer_close_kernel<float, 4>), dim3(rows), dim3(th), smem, s, (const float*)y, x, (float*)out_e, a);
    else DLI_LAUNCH("layer_close", (layer_close_kernel<float, 1>), dim3(rows), dim3(th), smem, s, (const float*)y, x, (float*)out_e, a);
  }
  return DLI_OK;
}

int dli_token_shift_ragged(const float* h, const float* shift, float* tail, const int32_t* row_ent, const int32_t* ent,
                           void* out, int rows, int d, int dt, dli_stream_t stream) {
  DLI_CHECK_ARG(h && shift && tail && row_ent && ent && out && d > 0, "dli_token_shift_ragged: null pointer or empty shape");
  DLI_CHECK_ARG((reinterpret_cast<uintptr_t>(ent) & 15u) == 0, "dli_token_shift_ragged: ent must be 16-byte aligned");
  DLI_CHECK_ARG(dt == 0 || dt == 1, "element type %d: 0 = bf16, 1 = float", dt);
  if (rows <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(rows, rows <= 64 ? (d + 1023) / 1024 : 1);
  if (dt == 0) DLI_LAUNCH("token_shift_ragged", token_shift_ragged_kernel<bf16>, grid, dim3(256), 0, s, h, shift, tail, row_ent, ent, (bf16*)out, d);
  else DLI_LAUNCH("token_shift_ragged", token_shift_ragged_kernel<float>, grid, dim3(256), 0, s, h, shift, tail, row_ent, ent, (float*)out, d);
  return DLI_OK;
}

}  // extern "C"
