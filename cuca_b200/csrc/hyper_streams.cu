// Several copies of the residual stream side by side (hyper-connections), X: [rows, S, E] in 32-bit:
//   spread_streams   every copy starts as the embedding output
//   streams_read     h = norm(sum_s r[s] X[s]) * w in the compute dtype (optionally of gathered rows)
//   streams_write    X'[t] = sum_s M[s, t] X[s] + o[t] y for all t from the old copies, in place; optionally the next
//                    sublayer's read of the new copies in the same launch
//   pair_norm_add    x (+)= c (norm(a) * wa + norm(b) * wb): two sublayer outputs normed apart, then joined
//   sigmoid_gate     a *= sigmoid(g), columns of two row-strided tensors
// All arithmetic is 32-bit; a row's reduction order depends on the width and on whether the launch has few rows.
#include "common.cuh"
#include <math.h>

namespace {

constexpr int MAX_STREAMS = 16;

// Blocks of NT threads take one row each; a thread works on V consecutive columns at a time (V = 4: 16-byte
// accesses, for widths that are multiples of four). Few rows (single tokens) get blocks of 1,024 threads, so that a
// row's few passes are not a chain of dependent loads in a handful of threads.
template <int NT>
__device__ __forceinline__ float block_total(float s, float* red) {
  s = warp_sum(s);
  __syncthreads();  // earlier readers of `red` are done
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < NT / 32; ++i) tot += red[i];
  return tot;
}

template <int V> struct Vec;
template <> struct Vec<1> { float v[1]; };
template <> struct alignas(16) Vec<4> { float v[4]; };
template <int V> __device__ __forceinline__ Vec<V> ld(const float* p) { return *reinterpret_cast<const Vec<V>*>(p); }
template <int V> __device__ __forceinline__ void st(float* p, const Vec<V>& x) { *reinterpret_cast<Vec<V>*>(p) = x; }
template <int V, typename TO> __device__ __forceinline__ void st_out(TO* p, const Vec<V>& x) {
#pragma unroll
  for (int k = 0; k < V; ++k) p[k] = from_f32<TO>(x.v[k]);
}

__global__ void spread_streams_kernel(const float* __restrict__ x, float* __restrict__ X, size_t n, int S, int E) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i / E, e = i % E;
    const float v = x[i];
    for (int s = 0; s < S; ++s) X[(row * S + s) * E + e] = v;
  }
}

// u[i..i+V) = sum_s r[s] X[row, s, i..i+V) (r null: every copy counts once)
template <int V>
__device__ __forceinline__ Vec<V> read_mix(const float* __restrict__ Xr, const float* rs, int S, int E, int i) {
  Vec<V> u;
#pragma unroll
  for (int k = 0; k < V; ++k) u.v[k] = 0.f;
  for (int s = 0; s < S; ++s) {
    const Vec<V> x = ld<V>(Xr + (size_t)s * E + i);
    const float c = rs ? rs[s] : 1.f;
#pragma unroll
    for (int k = 0; k < V; ++k) u.v[k] = fmaf(c, x.v[k], u.v[k]);
  }
  return u;
}

template <typename TO, int NT, int V>
__device__ __forceinline__ void read_row(const float* __restrict__ Xr, const float* rs, const float* __restrict__ w,
                                         TO* __restrict__ out, int S, int E, float eps, float* red) {
  float ss = 0.f;
  for (int i = threadIdx.x * V; i < E; i += NT * V) {
    const Vec<V> u = read_mix<V>(Xr, rs, S, E, i);
#pragma unroll
    for (int k = 0; k < V; ++k) ss = fmaf(u.v[k], u.v[k], ss);
  }
  const float inv = 1.f / sqrtf(block_total<NT>(ss, red) / (float)E + eps);
  for (int i = threadIdx.x * V; i < E; i += NT * V) {
    Vec<V> u = read_mix<V>(Xr, rs, S, E, i);
    const Vec<V> wv = ld<V>(w + i);
#pragma unroll
    for (int k = 0; k < V; ++k) u.v[k] = u.v[k] * inv * wv.v[k];
    st_out<V, TO>(out + i, u);
  }
}

template <typename TO, int NT, int V>
__global__ void __launch_bounds__(NT)
streams_read_kernel(const float* __restrict__ X, const float* __restrict__ r, const float* __restrict__ w,
                    TO* __restrict__ out, const int* __restrict__ rows, int S, int E, float eps) {
  __shared__ float red[NT / 32];
  __shared__ float rs[MAX_STREAMS];
  pdl_trigger();
  pdl_wait();
  if (r && threadIdx.x < S) rs[threadIdx.x] = r[threadIdx.x];
  __syncthreads();
  const size_t src = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
  read_row<TO, NT, V>(X + src * S * E, r ? rs : nullptr, w, out + (size_t)blockIdx.x * E, S, E, eps, red);
}

template <typename TO, bool NEXT, int NT, int V>
__global__ void __launch_bounds__(NT)
streams_write_kernel(float* __restrict__ X, const float* __restrict__ y, const float* __restrict__ M,
                     const float* __restrict__ o, const float* __restrict__ r2, const float* __restrict__ w2,
                     TO* __restrict__ out2, int S, int E, float eps) {
  __shared__ float red[NT / 32];
  __shared__ float ms[MAX_STREAMS * MAX_STREAMS], os[MAX_STREAMS], rs[MAX_STREAMS];
  pdl_trigger();
  pdl_wait();
  if (threadIdx.x < S * S) ms[threadIdx.x] = M[threadIdx.x];
  if (threadIdx.x < S) {
    os[threadIdx.x] = o[threadIdx.x];
    rs[threadIdx.x] = NEXT ? r2[threadIdx.x] : 0.f;
  }
  __syncthreads();
  float* Xr = X + (size_t)blockIdx.x * S * E;
  const float* yr = y + (size_t)blockIdx.x * E;
  float ss = 0.f;
  for (int i = threadIdx.x * V; i < E; i += NT * V) {
    Vec<V> old[MAX_STREAMS];
    for (int s = 0; s < S; ++s) old[s] = ld<V>(Xr + (size_t)s * E + i);
    const Vec<V> yi = ld<V>(yr + i);
    Vec<V> u2;
#pragma unroll
    for (int k = 0; k < V; ++k) u2.v[k] = 0.f;
    for (int t = 0; t < S; ++t) {
      Vec<V> nv;
#pragma unroll
      for (int k = 0; k < V; ++k) {
        float v = 0.f;
        for (int s = 0; s < S; ++s) v = fmaf(ms[s * S + t], old[s].v[k], v);
        nv.v[k] = fmaf(os[t], yi.v[k], v);
        if (NEXT) u2.v[k] = fmaf(rs[t], nv.v[k], u2.v[k]);
      }
      st<V>(Xr + (size_t)t * E + i, nv);
    }
    if (NEXT) {
#pragma unroll
      for (int k = 0; k < V; ++k) ss = fmaf(u2.v[k], u2.v[k], ss);
    }
  }
  if (!NEXT) return;
  // the next sublayer's read of the new copies: its sum of squares came with the write; the values are read back
  // (a thread re-reads only columns it wrote itself) and summed in the same order as in a read of their own
  const float inv = 1.f / sqrtf(block_total<NT>(ss, red) / (float)E + eps);
  for (int i = threadIdx.x * V; i < E; i += NT * V) {
    Vec<V> u = read_mix<V>(Xr, rs, S, E, i);
    const Vec<V> wv = ld<V>(w2 + i);
#pragma unroll
    for (int k = 0; k < V; ++k) u.v[k] = u.v[k] * inv * wv.v[k];
    st_out<V, TO>(out2 + (size_t)blockIdx.x * E + i, u);
  }
}

template <bool STORE>
__global__ void __launch_bounds__(256)
pair_norm_add_kernel(float* __restrict__ x, const float* __restrict__ a, const float* __restrict__ b,
                     const float* __restrict__ wa, const float* __restrict__ wb, float c, int E, float eps) {
  constexpr int NT = 256;
  __shared__ float red[NT / 32];
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.x;
  const float* ar = a + row * E;
  const float* br = b + row * E;
  float sa = 0.f, sb = 0.f;
  for (int i = threadIdx.x; i < E; i += NT) { sa = fmaf(ar[i], ar[i], sa); sb = fmaf(br[i], br[i], sb); }
  const float ia = 1.f / sqrtf(block_total<NT>(sa, red) / (float)E + eps);
  const float ib = 1.f / sqrtf(block_total<NT>(sb, red) / (float)E + eps);
  for (int i = threadIdx.x; i < E; i += NT) {
    const float v = c * (ar[i] * ia * wa[i] + br[i] * ib * wb[i]);
    x[row * E + i] = STORE ? v : x[row * E + i] + v;
  }
}

template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ a, int lda, const T* __restrict__ g, int ldg, int rows, int n) {
  pdl_trigger();
  pdl_wait();
  const size_t total = (size_t)rows * n;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / n, c = i % n;
    const float v = to_f32(a[r * lda + c]), z = to_f32(g[r * ldg + c]);
    a[r * lda + c] = from_f32<T>(v / (1.f + expf(-z)));
  }
}

// out[r, h, j ds + e] = parts[j][r, h, e] * sigmoid(g[r, h, j ds + e]) (g null: no gate): the slabs of an attention
// whose value heads were run as `split` narrower ones, joined again under the output gate
template <typename T>
__global__ void gate_merge_kernel(const T* __restrict__ parts, const T* __restrict__ g, int ldg, T* __restrict__ out,
                                  int rows, int nh, int dv, int split) {
  pdl_trigger();
  pdl_wait();
  const int ds = dv / split;
  const size_t total = (size_t)rows * nh * dv, slab = (size_t)rows * nh * ds;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / ((size_t)nh * dv);
    const int c = (int)(i % ((size_t)nh * dv)), h = c / dv, e = c % dv;
    float v = to_f32(parts[(e / ds) * slab + (r * nh + h) * ds + e % ds]);
    if (g) v /= 1.f + expf(-to_f32(g[r * ldg + c]));
    out[i] = from_f32<T>(v);
  }
}

int blocks_for(size_t n) {
  size_t b = (n + 255) / 256;
  return (int)(b < 1 ? 1 : (b > 4096 ? 4096 : b));
}

}  // namespace

CUCA_API int cuca_streams_max() { return MAX_STREAMS; }

CUCA_API int cuca_spread_streams(const float* x, float* X, int rows, int S, int E, cudaStream_t stream) {
  if (rows == 0) return 0;
  CUCA_REQUIRE(S >= 1 && E >= 1, "spread_streams: bad sizes copies=%d width=%d", S, E);
  const size_t n = (size_t)rows * E;
  cuca_launch(spread_streams_kernel, dim3(blocks_for(n)), dim3(256), 0, stream, true, x, X, n, S, E);
  CUCA_CHECK_LAUNCH("spread_streams");
  return 0;
}

// rows below this count get blocks of 1,024 threads
static bool few_rows(int rows) { return rows <= 256; }
static bool vec4(int E, const void* a, const void* b, const void* c, const void* d) {
  return E % 4 == 0 && (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c | (uintptr_t)d) & 15) == 0;
}

// out[j] = norm(sum_s r[s] X[rows ? rows[j] : j, s]) * w; r null: the plain sum of the copies
CUCA_API int cuca_streams_read(const float* X, const float* r, const float* w, void* out, int out_dtype,
                               const int* rows, int n_out, int S, int E, float eps, cudaStream_t stream) {
  if (n_out == 0) return 0;
  CUCA_REQUIRE(S >= 1 && S <= MAX_STREAMS && E >= 1, "streams_read: %d copies are outside 1..%d", S, MAX_STREAMS);
  CUCA_REQUIRE(out_dtype == CUCA_F32 || out_dtype == CUCA_BF16, "streams_read: unknown dtype %d", out_dtype);
  const bool v4 = vec4(E, X, w, nullptr, nullptr), big = few_rows(n_out);
#define SR(TO, NT, V)                                                                                            \
  cuca_launch(streams_read_kernel<TO, NT, V>, dim3(n_out), dim3(NT), 0, stream, true, X, r, w, (TO*)out, rows, S, E, eps)
#define SR_BY(TO)                                   \
  do {                                              \
    if (v4 && big) SR(TO, 1024, 4);                 \
    else if (v4) SR(TO, 256, 4);                    \
    else if (big) SR(TO, 1024, 1);                  \
    else SR(TO, 256, 1);                            \
  } while (0)
  if (out_dtype == CUCA_F32) SR_BY(float);
  else SR_BY(__nv_bfloat16);
#undef SR_BY
#undef SR
  CUCA_CHECK_LAUNCH("streams_read");
  return 0;
}

// X'[t] = sum_s M[s * S + t] X[s] + o[t] y; with out2: out2 = norm(sum_t r2[t] X'[t]) * w2
CUCA_API int cuca_streams_write(float* X, const float* y, const float* M, const float* o, const float* r2,
                                const float* w2, void* out2, int out_dtype, int rows, int S, int E, float eps,
                                cudaStream_t stream) {
  if (rows == 0) return 0;
  CUCA_REQUIRE(S >= 1 && S <= MAX_STREAMS && E >= 1, "streams_write: %d copies are outside 1..%d", S, MAX_STREAMS);
  CUCA_REQUIRE(out2 == nullptr || out_dtype == CUCA_F32 || out_dtype == CUCA_BF16, "streams_write: unknown dtype %d", out_dtype);
  const bool v4 = vec4(E, X, y, w2, nullptr), big = few_rows(rows);
#define SW(TO, NEXT, NT, V)                                                                                       \
  cuca_launch(streams_write_kernel<TO, NEXT, NT, V>, dim3(rows), dim3(NT), 0, stream, true, X, y, M, o, r2, w2, \
              (TO*)out2, S, E, eps)
#define SW_BY(TO, NEXT)                             \
  do {                                              \
    if (v4 && big) SW(TO, NEXT, 1024, 4);           \
    else if (v4) SW(TO, NEXT, 256, 4);              \
    else if (big) SW(TO, NEXT, 1024, 1);            \
    else SW(TO, NEXT, 256, 1);                      \
  } while (0)
  if (out2 == nullptr) SW_BY(float, false);
  else if (out_dtype == CUCA_F32) SW_BY(float, true);
  else SW_BY(__nv_bfloat16, true);
#undef SW_BY
#undef SW
  CUCA_CHECK_LAUNCH("streams_write");
  return 0;
}

CUCA_API int cuca_pair_norm_add(float* x, const float* a, const float* b, const float* wa, const float* wb, float c,
                                int store, int rows, int E, float eps, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (store)
    cuca_launch(pair_norm_add_kernel<true>, dim3(rows), dim3(256), 0, stream, true, x, a, b, wa, wb, c, E, eps);
  else
    cuca_launch(pair_norm_add_kernel<false>, dim3(rows), dim3(256), 0, stream, true, x, a, b, wa, wb, c, E, eps);
  CUCA_CHECK_LAUNCH("pair_norm_add");
  return 0;
}

CUCA_API int cuca_sigmoid_gate(void* a, int lda, const void* g, int ldg, int dtype, int rows, int n,
                               cudaStream_t stream) {
  if (rows == 0 || n == 0) return 0;
  const int blocks = blocks_for((size_t)rows * n);
  if (dtype == CUCA_F32)
    cuca_launch(sigmoid_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, true, (float*)a, lda, (const float*)g,
                ldg, rows, n);
  else if (dtype == CUCA_BF16)
    cuca_launch(sigmoid_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, true, (__nv_bfloat16*)a, lda,
                (const __nv_bfloat16*)g, ldg, rows, n);
  else
    CUCA_REQUIRE(false, "sigmoid_gate: unknown dtype %d", dtype);
  CUCA_CHECK_LAUNCH("sigmoid_gate");
  return 0;
}

CUCA_API int cuca_gate_merge(const void* parts, const void* g, int ldg, void* out, int dtype, int rows, int nh, int dv,
                             int split, cudaStream_t stream) {
  if (rows == 0) return 0;
  CUCA_REQUIRE(split >= 1 && dv % split == 0, "gate_merge: %d slabs do not divide value size %d", split, dv);
  const int blocks = blocks_for((size_t)rows * nh * dv);
  if (dtype == CUCA_F32)
    cuca_launch(gate_merge_kernel<float>, dim3(blocks), dim3(256), 0, stream, true, (const float*)parts, (const float*)g,
                ldg, (float*)out, rows, nh, dv, split);
  else if (dtype == CUCA_BF16)
    cuca_launch(gate_merge_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, true, (const __nv_bfloat16*)parts,
                (const __nv_bfloat16*)g, ldg, (__nv_bfloat16*)out, rows, nh, dv, split);
  else
    CUCA_REQUIRE(false, "gate_merge: unknown dtype %d", dtype);
  CUCA_CHECK_LAUNCH("gate_merge");
  return 0;
}
