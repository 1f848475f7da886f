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
// token shift and advances the slot's previous row.  dli_token_shift_ragged is the shift for steps with portions of
// prompts, on the normed rows.
#include "common.cuh"

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
};

// One CTA per row.  Pass 1 forms the new x (and its sum of squares), pass 2 the next norm from the rows just written.
template <typename E>
__global__ void __launch_bounds__(1024)
layer_close_kernel(const E* __restrict__ y, float* __restrict__ x, E* __restrict__ out_e, LayerClose a) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x, d = a.d;
  const size_t o = (size_t)row * d;
  const float iw = a.idw ? a.idw[row] : 0.f;
  float ss = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float v = x[o + c];
    if (y) {
      float t = pn_to_f(y[o + c]);
      if (a.bias) t += a.bias[c];
      if (a.idw) t = fmaf(iw, a.h_in[o + c], t);
      v = a.ls ? fmaf(a.ls[c], t, v) : v + t;
    }
    if (a.dwa) {
      a.xs[(size_t)a.n_prev * a.xs_stride + o + c] = v;
      float u = 0.f;
      for (int j = 0; j < a.n_prev; ++j) u = fmaf(a.dwa[j], a.xs[(size_t)j * a.xs_stride + o + c], u);
      v = fmaf(a.dwa[a.n_prev], v, u);
    }
    if (y || a.dwa) x[o + c] = v;
    ss = fmaf(v, v, ss);
  }
  if (!a.w_next) return;
  ss = pn_block_sum(ss, red);  // its barriers also order the writes of x above before the reads below
  const float r = 1.f / sqrtf(ss / d + a.eps);
  int slot = 0, pos = 0;
  if (a.shift) {
    const int4 e = reinterpret_cast<const int4*>(a.ent)[row];  // slot, first row (== row), 1, position
    slot = e.x; pos = e.w;
  }
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float h = x[o + c] * r * a.w_next[c];
    if (a.shift) {
      float* t = a.tail + (size_t)slot * d + c;
      const float prev = pos > 0 ? *t : 0.f;
      *t = h;
      h = fmaf(prev - h, a.shift[c], h);
    }
    if (a.out_f) a.out_f[o + c] = h;
    if (out_e) out_e[o + c] = pn_from_f<E>(h);
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
  if (rows <= 0) return DLI_OK;
  LayerClose a{bias, idw, h_in, ls, xs, xs_stride, n_prev, dwa, w_next, shift, tail, ent, out_f, eps, d};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int th = (rows <= 64 && d >= 2048) ? 1024 : 256;
  if (dt == 0) DLI_LAUNCH("layer_close", layer_close_kernel<bf16>, dim3(rows), dim3(th), 0, s, (const bf16*)y, x, (bf16*)out_e, a);
  else DLI_LAUNCH("layer_close", layer_close_kernel<float>, dim3(rows), dim3(th), 0, s, (const float*)y, x, (float*)out_e, a);
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
