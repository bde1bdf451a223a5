// Kernels around the 32-bit residual stream for blocks that norm a sublayer's input AND its output:
//   norm_shift      h = shift(norm(x)), the previous token's normed row mixed in, its last row kept per request
//   post_norm_add   x += norm(y) * g, and optionally f = norm(x) * g2 of the new row in the same pass
//   gelu, scale, concat2 (two streams side by side in the compute dtype, for a contraction over both)
// A norm's gain is a vector or a single number (gain_stride 1 or 0). All arithmetic is 32-bit, and a row's
// reduction order depends on the width alone, so its bits do not depend on the batch it is in.
#include "common.cuh"
#include <math.h>

namespace {

constexpr int NT = 256;

// sum of squares of a row, every thread gets the total; `red` holds 8 floats and may be reused after the call
__device__ __forceinline__ float row_sumsq(const float* __restrict__ xr, int E, float* red) {
  float s = 0.f;
  for (int i = threadIdx.x; i < E; i += NT) { float v = xr[i]; s = fmaf(v, v, s); }
  s = warp_sum(s);
  __syncthreads();  // earlier readers of `red` are done
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < NT / 32; ++i) tot += red[i];
  return tot;
}

// A normed value and the shift, rounded step by step: the previous token's value is the same bits whether it is
// computed here from its row or read back from where an earlier step kept it (no contraction across the two).
__device__ __forceinline__ float normed(float x, float inv, float g) { return __fmul_rn(__fmul_rn(x, inv), g); }
__device__ __forceinline__ float shifted(float h, float hp, float mix) { return __fmaf_rn(__fsub_rn(hp, h), mix, h); }

// Blocks 0..n_rows-1 take the rows that follow another row of their request in this step; blocks n_rows.. take one
// request each: its first row (whose predecessor is the request's kept row) and, after that, the new kept row.
// Only that block touches the request's kept row, reading before it writes.
template <typename TO>
__global__ void __launch_bounds__(NT)
norm_shift_kernel(const float* __restrict__ x, const float* __restrict__ gain, int gain_stride, float eps,
                  const float* __restrict__ mix, float* __restrict__ kept, TO* __restrict__ out,
                  const int* __restrict__ seq_of_row, const int* __restrict__ req_row0,
                  const int* __restrict__ req_count, const int* __restrict__ slots, int n_rows, int E) {
  __shared__ float red[NT / 32];
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x;
  if (b < n_rows) {
    const int seq = seq_of_row[b];
    if (seq < 0 || b == 0 || seq_of_row[b - 1] != seq) return;
    const float* xr = x + (size_t)b * E;
    const float* xp = xr - E;
    const float ir = rsqrtf(row_sumsq(xr, E, red) / (float)E + eps);
    const float ip = rsqrtf(row_sumsq(xp, E, red) / (float)E + eps);
    for (int i = threadIdx.x; i < E; i += NT) {
      const float g = gain[i * gain_stride];
      out[(size_t)b * E + i] = from_f32<TO>(shifted(normed(xr[i], ir, g), normed(xp[i], ip, g), mix[i]));
    }
    return;
  }
  const int q = b - n_rows;
  const int slot = slots[q], n = req_count[q], r0 = req_row0[q];
  if (slot < 0 || n <= 0) return;
  float* keep = kept + (size_t)slot * E;
  const float* xr = x + (size_t)r0 * E;
  const float* xl = x + (size_t)(r0 + n - 1) * E;
  const float ir = rsqrtf(row_sumsq(xr, E, red) / (float)E + eps);
  const float il = n == 1 ? ir : rsqrtf(row_sumsq(xl, E, red) / (float)E + eps);  // a single token: the same row
  for (int i = threadIdx.x; i < E; i += NT) {
    const float g = gain[i * gain_stride];
    out[(size_t)r0 * E + i] = from_f32<TO>(shifted(normed(xr[i], ir, g), keep[i], mix[i]));
    keep[i] = normed(xl[i], il, g);
  }
}

template <typename TO, bool NEXT>
__global__ void __launch_bounds__(NT)
post_norm_add_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ gain,
                     int gain_stride, const float* __restrict__ gain2, int gain2_stride, TO* __restrict__ out, int E,
                     float eps) {
  __shared__ float red[NT / 32];
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.x;
  float* xr = x + row * E;
  const float* yr = y + row * E;
  const float iy = rsqrtf(row_sumsq(yr, E, red) / (float)E + eps);
  for (int i = threadIdx.x; i < E; i += NT) xr[i] += yr[i] * iy * gain[i * gain_stride];
  if (!NEXT) return;
  // every thread reads back what it wrote itself and, in the reduction, what others wrote before the barrier inside
  __syncthreads();
  const float ix = rsqrtf(row_sumsq(xr, E, red) / (float)E + eps);
  for (int i = threadIdx.x; i < E; i += NT) out[row * E + i] = from_f32<TO>(xr[i] * ix * gain2[i * gain2_stride]);
}

__device__ __forceinline__ float gelu_of(float z, int tanh_form) {
  if (tanh_form) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  return 0.5f * z * (1.f + erff(z * 0.7071067811865476f));
}

// 16 bytes per thread and round where the tensor allows it (n_vec pieces), the rest value by value
template <typename T>
__global__ void gelu_kernel(T* __restrict__ a, size_t n, size_t n_vec, int tanh_form) {
  pdl_trigger();
  pdl_wait();
  constexpr int PER = 16 / sizeof(T);
  const size_t stride = (size_t)gridDim.x * blockDim.x, first = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (size_t i = first; i < n_vec; i += stride) {
    uint4 w = reinterpret_cast<uint4*>(a)[i];
    T* v = reinterpret_cast<T*>(&w);
#pragma unroll
    for (int k = 0; k < PER; ++k) v[k] = from_f32<T>(gelu_of(to_f32(v[k]), tanh_form));
    reinterpret_cast<uint4*>(a)[i] = w;
  }
  for (size_t i = n_vec * PER + first; i < n; i += stride) a[i] = from_f32<T>(gelu_of(to_f32(a[i]), tanh_form));
}

__global__ void scale_kernel(float* __restrict__ a, size_t n, float s) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) a[i] *= s;
}

template <typename TO>
__global__ void concat2_kernel(const float* __restrict__ a, const float* __restrict__ b, TO* __restrict__ out, int E) {
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.x;
  for (int i = threadIdx.x; i < E; i += blockDim.x) {
    out[row * 2 * E + i] = from_f32<TO>(a[row * E + i]);
    out[row * 2 * E + E + i] = from_f32<TO>(b[row * E + i]);
  }
}

inline unsigned flat_grid(size_t n, int threads) {
  size_t g = (n + threads - 1) / threads;
  return (unsigned)(g < 1 ? 1 : (g > 65535u * 8u ? 65535u * 8u : g));
}

}  // namespace

// out[r] = h[r] + (h[r-1] - h[r]) * mix with h = x * rsqrt(mean(x^2) + eps) * gain; the row before a request's first
// row of this step is kept[slot] (zeros for a new request), and kept[slot] becomes the request's last h of this step.
CUCA_API int cuca_norm_shift(const float* x, const float* gain, int gain_stride, float eps, const float* mix,
                             float* kept, void* out, int out_dtype, const int* seq_of_row, const int* req_row0,
                             const int* req_count, const int* slots, int n_rows, int n_seqs, int E,
                             cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CUCA_REQUIRE(E > 0 && n_seqs > 0, "norm_shift: bad sizes E=%d requests=%d", E, n_seqs);
  dim3 grid(n_rows + n_seqs);
  if (out_dtype == CUCA_F32)
    cuca_launch(norm_shift_kernel<float>, grid, dim3(NT), 0, stream, true, x, gain, gain_stride, eps, mix, kept,
                (float*)out, seq_of_row, req_row0, req_count, slots, n_rows, E);
  else if (out_dtype == CUCA_BF16)
    cuca_launch(norm_shift_kernel<__nv_bfloat16>, grid, dim3(NT), 0, stream, true, x, gain, gain_stride, eps, mix,
                kept, (__nv_bfloat16*)out, seq_of_row, req_row0, req_count, slots, n_rows, E);
  else
    CUCA_REQUIRE(false, "norm_shift: unknown dtype %d", out_dtype);
  CUCA_CHECK_LAUNCH("norm_shift");
  return 0;
}

// x += y * rsqrt(mean(y^2) + eps) * gain; with `out`: out = x * rsqrt(mean(x^2) + eps) * gain2 of the new x.
CUCA_API int cuca_post_norm_add(float* x, const float* y, const float* gain, int gain_stride, const float* gain2,
                                int gain2_stride, void* out, int out_dtype, int n_rows, int E, float eps,
                                cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CUCA_REQUIRE(E > 0, "post_norm_add: bad width %d", E);
  dim3 grid(n_rows);
  if (out == nullptr)
    cuca_launch(post_norm_add_kernel<float, false>, grid, dim3(NT), 0, stream, true, x, y, gain, gain_stride,
                (const float*)nullptr, 0, (float*)nullptr, E, eps);
  else if (out_dtype == CUCA_F32)
    cuca_launch(post_norm_add_kernel<float, true>, grid, dim3(NT), 0, stream, true, x, y, gain, gain_stride, gain2,
                gain2_stride, (float*)out, E, eps);
  else if (out_dtype == CUCA_BF16)
    cuca_launch(post_norm_add_kernel<__nv_bfloat16, true>, grid, dim3(NT), 0, stream, true, x, y, gain, gain_stride,
                gain2, gain2_stride, (__nv_bfloat16*)out, E, eps);
  else
    CUCA_REQUIRE(false, "post_norm_add: unknown dtype %d", out_dtype);
  CUCA_CHECK_LAUNCH("post_norm_add");
  return 0;
}

// a = gelu(a) in place: the exact form (erf), or the tanh form 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).
CUCA_API int cuca_gelu(void* a, int dtype, size_t n, int tanh_form, cudaStream_t stream) {
  if (n == 0) return 0;
  const bool aligned = (((size_t)a) & 15) == 0;
  if (dtype == CUCA_F32) {
    const size_t nv = aligned ? n / 4 : 0;
    cuca_launch(gelu_kernel<float>, dim3(flat_grid(nv > 0 ? nv : n, 256)), dim3(256), 0, stream, true, (float*)a, n, nv,
                tanh_form);
  } else if (dtype == CUCA_BF16) {
    const size_t nv = aligned ? n / 8 : 0;
    cuca_launch(gelu_kernel<__nv_bfloat16>, dim3(flat_grid(nv > 0 ? nv : n, 256)), dim3(256), 0, stream, true,
                (__nv_bfloat16*)a, n, nv, tanh_form);
  }
  else
    CUCA_REQUIRE(false, "gelu: unknown dtype %d", dtype);
  CUCA_CHECK_LAUNCH("gelu");
  return 0;
}

CUCA_API int cuca_scale(float* a, size_t n, float s, cudaStream_t stream) {
  if (n == 0) return 0;
  cuca_launch(scale_kernel, dim3(flat_grid(n, 256)), dim3(256), 0, stream, true, a, n, s);
  CUCA_CHECK_LAUNCH("scale");
  return 0;
}

// out[r] = [a[r] | b[r]] in the compute dtype (a, b: 32-bit [n_rows, E]).
CUCA_API int cuca_concat2(const float* a, const float* b, void* out, int out_dtype, int n_rows, int E,
                          cudaStream_t stream) {
  if (n_rows == 0) return 0;
  if (out_dtype == CUCA_F32)
    cuca_launch(concat2_kernel<float>, dim3(n_rows), dim3(256), 0, stream, true, a, b, (float*)out, E);
  else if (out_dtype == CUCA_BF16)
    cuca_launch(concat2_kernel<__nv_bfloat16>, dim3(n_rows), dim3(256), 0, stream, true, a, b, (__nv_bfloat16*)out, E);
  else
    CUCA_REQUIRE(false, "concat2: unknown dtype %d", out_dtype);
  CUCA_CHECK_LAUNCH("concat2");
  return 0;
}
