// Recurrent mixers: state carried from token to token in 32-bit, one slot per request.
//   mingru_scan        S = (1 - z) S + z c, gates from the current token alone
//   causal_conv        short convolution per channel over a request's tokens, its last inputs kept per request
//   ssm_scan           S = exp(-exp(A) dt) S + dt B x^T, y = S^T C + D x per head (scalar decay per head)
//   gated_group_norm   y * silu(z), RMS-normed in equal parts, times a weight
// A step brings each request a run of consecutive rows (req_row0, req_count); a kernel walks a request's rows in
// order from the state its slot holds and leaves the new state there. The order of the arithmetic along a sequence
// does not depend on where it was cut into steps.
#include "common.cuh"
#include <math.h>

namespace {

__device__ __forceinline__ float sigmoidf_(float v) { return 1.f / (1.f + expf(-v)); }
__device__ __forceinline__ float siluf_(float v) { return v / (1.f + expf(-v)); }

// zxg: [rows, 3 W] 32-bit (z, u and g before their activations, biases added). One thread per (request, channel).
template <typename TO>
__global__ void mingru_scan_kernel(const float* __restrict__ zxg, float* __restrict__ state, TO* __restrict__ out,
                                   const int* __restrict__ req_row0, const int* __restrict__ req_count,
                                   const int* __restrict__ slots, int W) {
  pdl_trigger();
  pdl_wait();
  const int q = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int slot = slots[q], n = req_count[q], r0 = req_row0[q];
  if (slot < 0 || n <= 0 || c >= W) return;
  float S = state[(size_t)slot * W + c];
  // eight tokens' inputs are requested before the first is used: the chain through S is short, the loads are not
  constexpr int U = 8;
  for (int t0 = 0; t0 < n; t0 += U) {
    float zr[U], ur[U], gr[U];
#pragma unroll
    for (int i = 0; i < U; ++i) {
      if (t0 + i < n) {
        const float* row = zxg + (size_t)(r0 + t0 + i) * 3 * W;
        zr[i] = row[c]; ur[i] = row[W + c]; gr[i] = row[2 * W + c];
      }
    }
#pragma unroll
    for (int i = 0; i < U; ++i) {
      if (t0 + i < n) {
        const float z = sigmoidf_(zr[i]);
        const float u = ur[i];
        const float cand = u >= 0.f ? u + 0.5f : sigmoidf_(u);
        S = (1.f - z) * S + z * cand;
        out[(size_t)(r0 + t0 + i) * W + c] = from_f32<TO>(S * siluf_(gr[i]));
      }
    }
  }
  state[(size_t)slot * W + c] = S;
}

// The same recurrence over long portions, cut into chunks of L tokens that run side by side: S_t = a_t S_(t-1) + b_t
// with a = 1 - z, b = z c composes, so a chunk is summed up as (product of a, its own end state from zero), the
// chunks' start states follow from those in one short pass per channel, and every chunk then runs from its start
// state. phase 0: chunk sums into carry[q][k][0..1][c]; phase 1: start states into carry[q][k][0][c], the request's
// state brought up to date; phase 2: the outputs. The start states are rounded differently than token by token.
template <typename TO>
__global__ void mingru_chunked_kernel(const float* __restrict__ zxg, float* __restrict__ state, float* __restrict__ carry,
                                      TO* __restrict__ out, const int* __restrict__ req_row0,
                                      const int* __restrict__ req_count, const int* __restrict__ slots, int W, int L,
                                      int max_chunks, int phase) {
  pdl_trigger();
  pdl_wait();
  const int q = blockIdx.z, k = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int slot = slots[q], n = req_count[q], r0 = req_row0[q];
  if (slot < 0 || n <= 0 || c >= W) return;
  const int n_chunks = (n + L - 1) / L;
  float* cq = carry + (size_t)q * max_chunks * 2 * W;
  if (phase == 1) {
    float S = state[(size_t)slot * W + c];
    for (int j = 0; j < n_chunks; ++j) {
      const float a = cq[(size_t)(2 * j) * W + c], b = cq[(size_t)(2 * j + 1) * W + c];
      cq[(size_t)(2 * j) * W + c] = S;
      S = fmaf(a, S, b);
    }
    state[(size_t)slot * W + c] = S;
    return;
  }
  if (k >= n_chunks) return;
  const int t1 = (k + 1) * L < n ? (k + 1) * L : n;
  float a = 1.f, S = phase == 0 ? 0.f : cq[(size_t)(2 * k) * W + c];
  for (int t = k * L; t < t1; ++t) {
    const float* row = zxg + (size_t)(r0 + t) * 3 * W;
    const float z = sigmoidf_(row[c]);
    const float u = row[W + c];
    const float cand = u >= 0.f ? u + 0.5f : sigmoidf_(u);
    S = (1.f - z) * S + z * cand;
    if (phase == 0) a *= 1.f - z;
    else out[(size_t)(r0 + t) * W + c] = from_f32<TO>(S * siluf_(row[2 * W + c]));
  }
  if (phase == 0) {
    cq[(size_t)(2 * k) * W + c] = a;
    cq[(size_t)(2 * k + 1) * W + c] = S;
  }
}

// in: 32-bit rows of stride ld_in, channel c at column col0 + c. kept: [slots, taps - 1, C] the inputs before the
// request's first row of this step (zeros for a new request). Blocks y < n_rows take rows that have taps - 1 rows of
// their own request before them in this step; blocks y >= n_rows take one request each: its first taps - 1 rows and
// then its new kept inputs (only that block touches them).
template <typename TW>
__global__ void causal_conv_kernel(const float* __restrict__ in, int ld_in, int col0, const TW* __restrict__ w,
                                   const TW* __restrict__ bias, float* __restrict__ kept, float* __restrict__ out,
                                   const int* __restrict__ seq_of_row, const int* __restrict__ req_row0,
                                   const int* __restrict__ req_count, const int* __restrict__ slots, int n_rows,
                                   int C, int taps) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int b = blockIdx.y;
  const int back = taps - 1;
  const TW* wc = w + (size_t)c * taps;
  const float b0 = bias ? to_f32(bias[c]) : 0.f;
  if (b < n_rows) {
    const int seq = seq_of_row[b];
    if (seq < 0 || b < back || (back > 0 && seq_of_row[b - back] != seq)) return;
    float acc = b0;
    for (int k = 0; k < taps; ++k)
      acc = fmaf(to_f32(wc[k]), in[(size_t)(b - back + k) * ld_in + col0 + c], acc);
    out[(size_t)b * C + c] = siluf_(acc);
    return;
  }
  if (back == 0) return;  // a one-tap convolution keeps nothing and every row was a plain row
  const int q = b - n_rows;
  const int slot = slots[q], n = req_count[q], r0 = req_row0[q];
  if (slot < 0 || n <= 0) return;
  float* keep = kept + (size_t)slot * back * C;
  // val(m): the input m rows after the request's first row of this step; m < 0 reaches into the kept inputs
  auto val = [&](int m) -> float {
    return m < 0 ? keep[(size_t)(m + back) * C + c] : in[(size_t)(r0 + m) * ld_in + col0 + c];
  };
  const int head = n < back ? n : back;
  for (int j = 0; j < head; ++j) {
    float acc = b0;
    for (int k = 0; k < taps; ++k) acc = fmaf(to_f32(wc[k]), val(j - back + k), acc);
    out[(size_t)(r0 + j) * C + c] = siluf_(acc);
  }
  // new kept inputs: the last `back` inputs of the sequence so far. Ascending k reads entries at or after the one
  // it writes (old entry n + k for the new entry k), so nothing is overwritten before it is read.
  for (int k = 0; k < back; ++k) {
    const float v = val(n - back + k);
    keep[(size_t)k * C + c] = v;
  }
}

constexpr int SSM_MAXR = 32;  // state values a thread holds

// an asynchronous copy of 4 or 16 bytes from global to shared memory
__device__ __forceinline__ void cp_async_f(float* dst, const float* src, int bytes) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  if (bytes == 16) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
  else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}

// One block per (head, request, run of PB value columns). Thread (p, s): value column p, state rows s, s + NS,
// s + 2 NS, ... (neighbouring threads read neighbouring shared-memory banks). state: [slots, H, P, N]. xbc: 32-bit [rows, H P + 2 G N] after the convolution (x | B | C); dt_raw: rows of stride ld_dt,
// head h at column dt_col + h, before bias and softplus.
// NR: state rows a thread holds at most. NST: threads per value column when that is known at compile time and divides
// the state evenly into NR rows each (the recurrence's loop is then free of index arithmetic and predicates: the
// kernel is bound by how many instructions it issues); 0: the number comes at run time and rows are checked.
template <int NR, int NST>
__global__ void ssm_scan_kernel(const float* __restrict__ xbc, const float* __restrict__ dt_raw, int ld_dt, int dt_col,
                                const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                const float* __restrict__ d_skip, float* __restrict__ state, float* __restrict__ y,
                                const int* __restrict__ req_row0, const int* __restrict__ req_count,
                                const int* __restrict__ slots, int H, int P, int N, int G, int NS_rt, int TC,
                                int PB) {
  const int NS = NST ? NST : NS_rt;
  extern __shared__ __align__(16) float sm[];
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.x, q = blockIdx.y;
  const int slot = slots[q], n = req_count[q], r0 = req_row0[q];
  if (slot < 0 || n <= 0) return;
  const int p_raw = blockIdx.z * PB + threadIdx.x / NS, s = threadIdx.x % NS;
  const bool live = threadIdx.x / NS < PB && p_raw < P;
  const int p = live ? p_raw : P - 1;
  const int g = h / (H / G);
  const int C = H * P + 2 * G * N;
  float S[NR];
  float* st = state + (((size_t)slot * H + h) * P + p) * N;
#pragma unroll
  for (int i = 0; i < NR; ++i) S[i] = (NST || s + i * NS < N) ? st[s + i * NS] : 0.f;
  const float A = -expf(a_log[h]);
  const float bias = dt_bias[h], D = d_skip[h];
  // A token's inputs in shared memory: B [N], C [N], x [P], step size, decay; `per` floats, a multiple of four.
  // Two runs of TC tokens: the next run's copies (cp.async) are in flight while this one is worked through.
  const int span = 2 * N + P;
  const int per = (span + 2 + 3) & ~3;
  const bool vec4 = ((N | P | (H * P)) & 3) == 0;
  auto stage = [&](int t0, int buf) {
    const int nt = n - t0 < TC ? n - t0 : TC;
    float* dst = sm + (size_t)buf * TC * per;
    if (vec4) {
      const int units = span >> 2;
      for (int e = threadIdx.x; e < nt * units; e += blockDim.x) {
        const int tt = e / units, i = (e - tt * units) << 2;
        const int col = i < 2 * N ? H * P + g * N + i + (i >= N ? (G - 1) * N : 0) : h * P + (i - 2 * N);
        cp_async_f(dst + tt * per + i, xbc + (size_t)(r0 + t0 + tt) * C + col, 16);
      }
    } else {
      for (int e = threadIdx.x; e < nt * span; e += blockDim.x) {
        const int tt = e / span, i = e - tt * span;
        const int col = i < 2 * N ? H * P + g * N + i + (i >= N ? (G - 1) * N : 0) : h * P + (i - 2 * N);
        cp_async_f(dst + tt * per + i, xbc + (size_t)(r0 + t0 + tt) * C + col, 4);
      }
    }
    for (int e = threadIdx.x; e < nt; e += blockDim.x)
      cp_async_f(dst + e * per + span, dt_raw + (size_t)(r0 + t0 + e) * ld_dt + dt_col + h, 4);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  stage(0, 0);
  for (int t0 = 0, run = 0; t0 < n; t0 += TC, ++run) {
    const int nt = n - t0 < TC ? n - t0 : TC;
    float* cur = sm + (size_t)(run & 1) * TC * per;
    if (t0 + TC < n) {
      stage(t0 + TC, (run & 1) ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x < nt) {  // step size and decay of every token of the run, once
      float* in = cur + threadIdx.x * per;
      const float raw = in[span] + bias;
      const float dt = raw > 20.f ? raw : log1pf(expf(raw));
      in[span] = dt;
      in[span + 1] = expf(A * dt);
    }
    __syncthreads();
    // (tokens only hang together through one multiply-add per state value: four of them are worked through at once)
#pragma unroll 4
    for (int tt = 0; tt < nt; ++tt) {
      const float* in = cur + tt * per;
      const float dt = in[span], decay = in[span + 1];
      const float x = in[2 * N + p];
      const float* Br = in + s;
      const float* Cr = in + N + s;
      const float dx = dt * x;
      // four partial sums, in an order that depends on the sizes alone
      float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < NR; ++i) {
        if (NST || s + i * NS < N) {
          S[i] = fmaf(decay, S[i], dx * Br[i * NS]);
          part[i & 3] = fmaf(S[i], Cr[i * NS], part[i & 3]);
        }
      }
      float acc = (part[0] + part[1]) + (part[2] + part[3]);
      for (int o = NS >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (live && s == 0) y[(size_t)(r0 + t0 + tt) * (H * P) + h * P + p] = acc + D * x;
    }
    __syncthreads();  // this run is read to the end before the run after next is copied over it
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NR; ++i)
      if (NST || s + i * NS < N) st[s + i * NS] = S[i];
  }
}

// One block per (row, part). v = y * silu(z); out = v * rsqrt(mean over the part (v^2) + eps) * w.
template <typename TW, typename TO>
__global__ void __launch_bounds__(256)
gated_group_norm_kernel(const float* __restrict__ y, const float* __restrict__ z, int ld_z, const TW* __restrict__ w,
                        TO* __restrict__ out, int inner, int part, float eps) {
  __shared__ float red[8];
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.y;
  const int c0 = blockIdx.x * part;
  float s = 0.f;
  // parts of up to 4096 values stay in registers between the two passes (all loads of the row in flight together)
  constexpr int KEEP = 16;
  float kept[KEEP];
  const bool keep = part <= KEEP * 256;
  if (keep) {
    float yv[KEEP], zv[KEEP];
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
      const int i = threadIdx.x + k * 256;
      if (i < part) { yv[k] = y[row * inner + c0 + i]; zv[k] = z[row * ld_z + c0 + i]; }
    }
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
      const int i = threadIdx.x + k * 256;
      kept[k] = i < part ? yv[k] * siluf_(zv[k]) : 0.f;
      s = fmaf(kept[k], kept[k], s);
    }
  } else {
    for (int i = threadIdx.x; i < part; i += 256) {
      const float v = y[row * inner + c0 + i] * siluf_(z[row * ld_z + c0 + i]);
      s = fmaf(v, v, s);
    }
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float inv = rsqrtf(tot / (float)part + eps);
  if (keep) {
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
      const int i = threadIdx.x + k * 256;
      if (i < part) out[row * inner + c0 + i] = from_f32<TO>(kept[k] * inv * to_f32(w[c0 + i]));
    }
    return;
  }
  for (int i = threadIdx.x; i < part; i += 256) {
    const float v = y[row * inner + c0 + i] * siluf_(z[row * ld_z + c0 + i]);
    out[row * inner + c0 + i] = from_f32<TO>(v * inv * to_f32(w[c0 + i]));
  }
}

}  // namespace

CUCA_API int cuca_mingru_scan(const float* zxg, float* state, void* out, int out_dtype, const int* req_row0,
                              const int* req_count, const int* slots, int n_seqs, int W, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  CUCA_REQUIRE(W > 0 && n_seqs <= 65535, "mingru_scan: bad sizes W=%d requests=%d", W, n_seqs);
  dim3 grid((W + 127) / 128, n_seqs);
  if (out_dtype == CUCA_F32)
    cuca_launch(mingru_scan_kernel<float>, grid, dim3(128), 0, stream, true, zxg, state, (float*)out, req_row0,
                req_count, slots, W);
  else if (out_dtype == CUCA_BF16)
    cuca_launch(mingru_scan_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, true, zxg, state, (__nv_bfloat16*)out,
                req_row0, req_count, slots, W);
  else
    CUCA_REQUIRE(false, "mingru_scan: unknown dtype %d", out_dtype);
  CUCA_CHECK_LAUNCH("mingru_scan");
  return 0;
}

// Long portions in chunks of `L` tokens side by side (see the kernel). carry: [n_seqs, max_chunks, 2, W] 32-bit
// scratch, max_chunks >= ceil(longest portion / L).
CUCA_API int cuca_mingru_scan_chunked(const float* zxg, float* state, float* carry, void* out, int out_dtype,
                                      const int* req_row0, const int* req_count, const int* slots, int n_seqs, int W,
                                      int L, int max_chunks, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  CUCA_REQUIRE(W > 0 && L > 0 && max_chunks > 0 && n_seqs <= 65535 && max_chunks <= 65535,
               "mingru_scan_chunked: bad sizes W=%d L=%d chunks=%d requests=%d", W, L, max_chunks, n_seqs);
  for (int phase = 0; phase < 3; ++phase) {
    dim3 grid((W + 127) / 128, phase == 1 ? 1 : max_chunks, n_seqs);
    if (out_dtype == CUCA_F32)
      cuca_launch(mingru_chunked_kernel<float>, grid, dim3(128), 0, stream, true, zxg, state, carry, (float*)out,
                  req_row0, req_count, slots, W, L, max_chunks, phase);
    else if (out_dtype == CUCA_BF16)
      cuca_launch(mingru_chunked_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, true, zxg, state, carry,
                  (__nv_bfloat16*)out, req_row0, req_count, slots, W, L, max_chunks, phase);
    else
      CUCA_REQUIRE(false, "mingru_scan_chunked: unknown dtype %d", out_dtype);
    CUCA_CHECK_LAUNCH("mingru_scan_chunked");
  }
  return 0;
}

CUCA_API int cuca_causal_conv(const float* in, int ld_in, int col0, const void* w, const void* bias, int w_dtype,
                              float* kept, float* out, const int* seq_of_row, const int* req_row0,
                              const int* req_count, const int* slots, int n_rows, int n_seqs, int C, int taps,
                              cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CUCA_REQUIRE(C > 0 && taps >= 1, "causal_conv: bad sizes channels=%d taps=%d", C, taps);
  CUCA_REQUIRE(n_rows + n_seqs <= 65535, "causal_conv: %d rows in one step exceed the launch limit", n_rows);
  dim3 grid((C + 127) / 128, n_rows + n_seqs);
  if (w_dtype == CUCA_F32)
    cuca_launch(causal_conv_kernel<float>, grid, dim3(128), 0, stream, true, in, ld_in, col0, (const float*)w,
                (const float*)bias, kept, out, seq_of_row, req_row0, req_count, slots, n_rows, C, taps);
  else if (w_dtype == CUCA_BF16)
    cuca_launch(causal_conv_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, true, in, ld_in, col0,
                (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias, kept, out, seq_of_row, req_row0, req_count, slots,
                n_rows, C, taps);
  else
    CUCA_REQUIRE(false, "causal_conv: unknown dtype %d", w_dtype);
  CUCA_CHECK_LAUNCH("causal_conv");
  return 0;
}

// How the state rows of a head are dealt to threads: (threads per value column, state rows per thread).
CUCA_API int cuca_ssm_scan_split(int P, int N, int* ns_out, int* nr_out) {
  int ns = 1;
  while ((N + ns - 1) / ns > SSM_MAXR && ns < 32) ns <<= 1;
  if ((N + ns - 1) / ns > SSM_MAXR) return 1;
  while (ns < 16 && ns * 4 <= N) ns <<= 1;  // at least four state rows a thread, at most sixteen threads a column
  *ns_out = ns;
  *nr_out = (N + ns - 1) / ns;
  return 0;
}

CUCA_API int cuca_ssm_scan(const float* xbc, const float* dt_raw, int ld_dt, int dt_col, const float* dt_bias,
                           const float* a_log, const float* d_skip, float* state, float* y, const int* req_row0,
                           const int* req_count, const int* slots, int n_seqs, int H, int P, int N, int G,
                           cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  CUCA_REQUIRE(H > 0 && P > 0 && N > 0 && G > 0 && H % G == 0, "ssm_scan: bad sizes heads=%d vdim=%d state=%d groups=%d",
               H, P, N, G);
  CUCA_REQUIRE(n_seqs <= 65535, "ssm_scan: %d requests exceed the launch limit", n_seqs);
  int ns, nr;
  CUCA_REQUIRE(cuca_ssm_scan_split(P, N, &ns, &nr) == 0, "ssm_scan: state size %d exceeds %d", N, 32 * SSM_MAXR);
  // value columns of a block: what fills 128 threads, so that a head's columns spread over several SMs
  int pb = 128 / ns;
  pb = pb < 1 ? 1 : (pb > P ? P : pb);
  const int threads = (pb * ns + 31) / 32 * 32;
  // tokens whose inputs are staged together: two runs of as many as 44 KB of shared memory hold, 16 at most
  const int per = (2 * N + P + 2 + 3) & ~3;
  int tc = 45056 / (2 * per * 4);
  tc = tc > 16 ? 16 : tc;
  CUCA_REQUIRE(tc >= 1, "ssm_scan: state size %d and value size %d exceed a token's shared memory", N, P);
#define SSM(NR, NST)                                                                                              \
  cuca_launch(ssm_scan_kernel<NR, NST>, dim3(H, n_seqs, (P + pb - 1) / pb), dim3(threads), (size_t)2 * tc * per * 4, \
              stream, true, xbc, dt_raw, ld_dt, dt_col, dt_bias, a_log, d_skip, state, y, req_row0, req_count, slots, \
              H, P, N, G, ns, tc, pb)
#define SSM_BY_NS(NR)                                     \
  do {                                                    \
    if (!exact) SSM(NR, 0);                               \
    else if (ns == 16) SSM(NR, 16);                       \
    else if (ns == 8) SSM(NR, 8);                         \
    else if (ns == 4) SSM(NR, 4);                         \
    else if (ns == 2) SSM(NR, 2);                         \
    else SSM(NR, 1);                                      \
  } while (0)
  // the state divides evenly into a row count the kernels are compiled for: the form without checks
  const bool exact = N % ns == 0 && (nr == 4 || nr == 8 || nr == 16 || nr == 32);
  if (nr <= 4) SSM_BY_NS(4);
  else if (nr <= 8) SSM_BY_NS(8);
  else if (nr <= 16) SSM_BY_NS(16);
  else SSM_BY_NS(32);
#undef SSM_BY_NS
#undef SSM
  CUCA_CHECK_LAUNCH("ssm_scan");
  return 0;
}

CUCA_API int cuca_gated_group_norm(const float* y, const float* z, int ld_z, const void* w, int w_dtype, void* out,
                                   int out_dtype, int n_rows, int inner, int parts, float eps, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CUCA_REQUIRE(parts > 0 && inner % parts == 0, "gated_group_norm: %d parts do not divide %d", parts, inner);
  CUCA_REQUIRE(n_rows <= 65535, "gated_group_norm: %d rows exceed the launch limit", n_rows);
  dim3 grid(parts, n_rows);
  const int part = inner / parts;
#define GGN(TW, TO)                                                                                               \
  cuca_launch(gated_group_norm_kernel<TW, TO>, grid, dim3(256), 0, stream, true, y, z, ld_z, (const TW*)w, (TO*)out, \
              inner, part, eps)
  if (w_dtype == CUCA_F32 && out_dtype == CUCA_F32) GGN(float, float);
  else if (w_dtype == CUCA_BF16 && out_dtype == CUCA_BF16) GGN(__nv_bfloat16, __nv_bfloat16);
  else if (w_dtype == CUCA_F32 && out_dtype == CUCA_BF16) GGN(float, __nv_bfloat16);
  else CUCA_REQUIRE(false, "gated_group_norm: unsupported dtypes %d/%d", w_dtype, out_dtype);
#undef GGN
  CUCA_CHECK_LAUNCH("gated_group_norm");
  return 0;
}
