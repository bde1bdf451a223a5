// A routed feed-forward: every token goes to the `top` experts with the largest router logits.
//   moe_route        per token: the chosen experts (largest logit first, the lower number on a tie), their weights
//                    (a softmax of just those logits) and, optionally, the weights spread over all experts
//   moe_act_dense    a[t, e, f] = relu(u[t, e, f])^2 * weight[t, e]: all experts' up-projections at once, the ones a
//                    token did not choose weighted 0, so that one contraction over (e, f) is the weighted sum
//   moe_up_sparse / moe_down_sparse   few tokens: only the chosen experts' weights are read, a warp per output
// Routing arithmetic is 32-bit. A token's experts are summed in a fixed order, whatever else is in the batch.
#include "common.cuh"
#include <math.h>

namespace {

constexpr int MAX_TOP = 32;
constexpr int MAX_EXPERTS = 1024;

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, int T, int E, int top, int* __restrict__ idx,
                 float* __restrict__ wts, float* __restrict__ dense) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  const float* z = logits + (size_t)t * E;
  unsigned taken = 0;  // bit j: this lane's expert lane + 32 j is chosen already
  float my_z = 0.f;    // lane j keeps the j-th chosen logit
  int my_e = 0;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int be = 0x7fffffff;
    for (int k = 0; lane + 32 * k < E; ++k) {
      const int e = lane + 32 * k;
      float v = z[e];
      v = v == v ? v : -INFINITY;  // a row of padding may hold anything: every lane must still see one order
      if (!((taken >> k) & 1u) && (v > best || (v == best && e < be) || be == 0x7fffffff)) { best = v; be = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (oe != 0x7fffffff && (be == 0x7fffffff || ov > best || (ov == best && oe < be))) { best = ov; be = oe; }
    }
    if (be < E && (be & 31) == lane) taken |= 1u << (be >> 5);
    if (lane == j) { my_z = best; my_e = be < E ? be : 0; }
  }
  const float zmax = __shfl_sync(0xffffffffu, my_z, 0);
  const float p = lane < top ? expf(my_z - zmax) : 0.f;
  const float w = p / warp_sum(p);
  if (dense)
    for (int e = lane; e < E; e += 32) dense[(size_t)t * E + e] = 0.f;
  __syncwarp();
  if (lane < top) {
    idx[(size_t)t * top + lane] = my_e;
    wts[(size_t)t * top + lane] = w;
    if (dense) dense[(size_t)t * E + my_e] = w;
  }
}

template <typename T>
__global__ void moe_act_dense_kernel(const T* __restrict__ u, const float* __restrict__ dense, T* __restrict__ a,
                                     size_t n, int E, int F) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / ((size_t)E * F);
    const int e = (int)((i / F) % E);
    const float w = dense[t * E + e];
    const float v = fmaxf(to_f32(u[i]), 0.f);
    a[i] = from_f32<T>(w == 0.f ? 0.f : v * v * w);
  }
}

// A warp's dot product of two rows of n values: 16 bytes a lane at a time where the rows allow it.
__device__ __forceinline__ float warp_dot(const float* w, const float* x, int n, int lane) {
  float acc = 0.f;
  for (int i = lane; i < n; i += 32) acc = fmaf(w[i], x[i], acc);
  return warp_sum(acc);
}
__device__ __forceinline__ float warp_dot(const __nv_bfloat16* w, const __nv_bfloat16* x, int n, int lane) {
  float acc = 0.f;
  if (n % 8 == 0 && ((((uintptr_t)w) | ((uintptr_t)x)) & 15) == 0) {
    for (int i = lane * 8; i < n; i += 256) {
      const uint4 a = *reinterpret_cast<const uint4*>(w + i), b = *reinterpret_cast<const uint4*>(x + i);
      const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 fa = __bfloat1622float2(pa[k]), fb = __bfloat1622float2(pb[k]);
        acc = fmaf(fa.x, fb.x, acc);
        acc = fmaf(fa.y, fb.y, acc);
      }
    }
  } else {
    for (int i = lane; i < n; i += 32) acc = fmaf(__bfloat162float(w[i]), __bfloat162float(x[i]), acc);
  }
  return warp_sum(acc);
}

// a[pair, f] = relu(W_up[e(pair)][f] . h[t])^2 * weight(pair); pair = t * top + j. W_up: [E F, K].
template <typename T>
__global__ void __launch_bounds__(256)
moe_up_sparse_kernel(const T* __restrict__ h, const T* __restrict__ w_up, const int* __restrict__ idx,
                     const float* __restrict__ wts, T* __restrict__ a, int top, int F, int K) {
  pdl_trigger();
  pdl_wait();
  const int pair = blockIdx.y, f = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (f >= F) return;
  const int e = idx[pair];
  const T* wr = w_up + ((size_t)e * F + f) * K;
  const T* hr = h + (size_t)(pair / top) * K;
  const float acc = warp_dot(wr, hr, K, lane);
  if (lane == 0) {
    const float v = fmaxf(acc, 0.f);
    a[(size_t)pair * F + f] = from_f32<T>(v * v * wts[pair]);
  }
}

// y[t, o] (+)= sum_j W_down[o, e(t, j) F ..] . a[t * top + j]; W_down: [N, E F]
template <typename T>
__global__ void __launch_bounds__(256)
moe_down_sparse_kernel(const T* __restrict__ a, const T* __restrict__ w_down, const int* __restrict__ idx,
                       float* __restrict__ y, int store, int top, int F, int E, int N) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.y, o = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (o >= N) return;
  float acc = 0.f;
  for (int j = 0; j < top; ++j) {
    const int e = idx[(size_t)t * top + j];
    const T* wr = w_down + (size_t)o * E * F + (size_t)e * F;
    const T* ar = a + ((size_t)t * top + j) * F;
    acc += warp_dot(wr, ar, F, lane);
  }
  if (lane == 0) y[(size_t)t * N + o] = store ? acc : y[(size_t)t * N + o] + acc;
}

}  // namespace

CUCA_API int cuca_moe_max_experts() { return MAX_EXPERTS; }

CUCA_API int cuca_moe_route(const float* logits, int T, int E, int top, int* idx, float* wts, float* dense,
                            cudaStream_t stream) {
  if (T == 0) return 0;
  CUCA_REQUIRE(E >= 1 && E <= MAX_EXPERTS && top >= 1 && top <= E && top <= MAX_TOP,
               "moe_route: %d of %d experts is outside what the kernel takes (experts <= %d, chosen <= %d)", top, E,
               MAX_EXPERTS, MAX_TOP);
  cuca_launch(moe_route_kernel, dim3((T + 3) / 4), dim3(128), 0, stream, true, logits, T, E, top, idx, wts, dense);
  CUCA_CHECK_LAUNCH("moe_route");
  return 0;
}

CUCA_API int cuca_moe_act_dense(const void* u, const float* dense, void* a, int dtype, int T, int E, int F,
                                cudaStream_t stream) {
  if (T == 0) return 0;
  const size_t n = (size_t)T * E * F;
  size_t blocks = (n + 255) / 256;
  blocks = blocks > 8192 ? 8192 : blocks;
  if (dtype == CUCA_F32)
    cuca_launch(moe_act_dense_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, true, (const float*)u, dense,
                (float*)a, n, E, F);
  else if (dtype == CUCA_BF16)
    cuca_launch(moe_act_dense_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, stream, true,
                (const __nv_bfloat16*)u, dense, (__nv_bfloat16*)a, n, E, F);
  else
    CUCA_REQUIRE(false, "moe_act_dense: unknown dtype %d", dtype);
  CUCA_CHECK_LAUNCH("moe_act_dense");
  return 0;
}

CUCA_API int cuca_moe_sparse(const void* h, const void* w_up, const void* w_down, const int* idx, const float* wts,
                             void* a, float* y, int store, int dtype, int T, int top, int E, int F, int K, int N,
                             cudaStream_t stream) {
  if (T == 0) return 0;
  CUCA_REQUIRE(T * top <= 65535 && T <= 65535, "moe_sparse: %d tokens exceed the launch limit", T);
  if (dtype == CUCA_F32) {
    cuca_launch(moe_up_sparse_kernel<float>, dim3((F + 7) / 8, T * top), dim3(256), 0, stream, true, (const float*)h,
                (const float*)w_up, idx, wts, (float*)a, top, F, K);
    CUCA_CHECK_LAUNCH("moe_up_sparse");
    cuca_launch(moe_down_sparse_kernel<float>, dim3((N + 7) / 8, T), dim3(256), 0, stream, true, (const float*)a,
                (const float*)w_down, idx, y, store, top, F, E, N);
  } else if (dtype == CUCA_BF16) {
    cuca_launch(moe_up_sparse_kernel<__nv_bfloat16>, dim3((F + 7) / 8, T * top), dim3(256), 0, stream, true,
                (const __nv_bfloat16*)h, (const __nv_bfloat16*)w_up, idx, wts, (__nv_bfloat16*)a, top, F, K);
    CUCA_CHECK_LAUNCH("moe_up_sparse");
    cuca_launch(moe_down_sparse_kernel<__nv_bfloat16>, dim3((N + 7) / 8, T), dim3(256), 0, stream, true,
                (const __nv_bfloat16*)a, (const __nv_bfloat16*)w_down, idx, y, store, top, F, E, N);
  } else {
    CUCA_REQUIRE(false, "moe_sparse: unknown dtype %d", dtype);
  }
  CUCA_CHECK_LAUNCH("moe_down_sparse");
  return 0;
}
