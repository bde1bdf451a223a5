// Mixers whose per-request state is a matrix per head, S [key channels, value columns], carried in 32-bit:
//   delta_scan      the delta rule with a decay per key channel:
//                     S <- g * S (rows);  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//   mlstm_scan      a matrix memory with exponential gates and a running maximum m (0 at the start):
//                     m' = max(f + m, i);  S <- e^(f + m - m') S + e^(i - m') k v^T;  n likewise from k alone;
//                     o = S^T q / (max(|n . q|, e^(-m')) + 1e-6)
//   head_norm_gate  out = o / rms(o) per head, times a weight, times sigmoid(gate)
// A block takes one (head, request, run of value columns) and walks the request's rows of the step in order from the
// state its slot holds, leaving the new state there. A value column's state rows live in the registers of NS
// neighbouring threads (thread s holds rows s, s + NS, ...); a token's vectors are staged in shared memory a few
// tokens at a time. The arithmetic of a token does not depend on where the sequence was cut into steps or chunks.
#include "common.cuh"
#include <math.h>

namespace {

constexpr int MAXR = 32;  // state rows a thread holds at most

__device__ __forceinline__ float sigmoidf_(float v) { return 1.f / (1.f + expf(-v)); }
__device__ __forceinline__ float softplusf_(float v) { return v > 20.f ? v : log1pf(expf(v)); }
__device__ __forceinline__ float log_sigmoidf_(float v) { return v < 0.f ? v - log1pf(expf(v)) : -log1pf(expf(-v)); }

// sum over the NS neighbouring threads of a value column (NS a power of two, at most 32)
__device__ __forceinline__ float group_sum(float v, int NS) {
  for (int o = NS >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// qkv: 32-bit rows of stride ld (after the short convolution and its activation): q heads at column 0 (G heads of
// d), k heads at column G d, v heads at column 2 G d (H heads of dv). a_raw: [rows, H d] decay pre-activations;
// b_raw: rows of stride ld_b, head h at column b_col + h. state: [slots, H, dv, d]. out: [rows, H dv].
template <int NR>
__global__ void delta_scan_kernel(const float* __restrict__ qkv, int ld, const float* __restrict__ a_raw,
                                  const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                  const float* __restrict__ b_raw, int ld_b, int b_col, float* __restrict__ state,
                                  float* __restrict__ out, const int* __restrict__ req_row0,
                                  const int* __restrict__ req_count, const int* __restrict__ slots, int H, int G,
                                  int d, int dv, int NS, int PB, int TC) {
  extern __shared__ __align__(16) float sm[];
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.x, rq = blockIdx.y;
  const int slot = slots[rq], n = req_count[rq], r0 = req_row0[rq];
  if (slot < 0 || n <= 0) return;
  const int kvh = h / (H / G);
  const int dp = NS * NR;  // key channels padded to what the threads hold
  float* sq = sm;                      // [TC][dp]
  float* sk = sq + (size_t)TC * dp;    // [TC][dp]
  float* sg = sk + (size_t)TC * dp;    // [TC][dp]
  float* sv = sg + (size_t)TC * dp;    // [TC][PB]
  float* sb = sv + (size_t)TC * PB;    // [TC]
  const int col_local = threadIdx.x / NS, s = threadIdx.x % NS;
  const int col = blockIdx.z * PB + col_local;
  const bool live = col_local < PB && col < dv;
  float S[NR];
  float* st = state + (((size_t)slot * H + h) * dv + (live ? col : 0)) * d;
#pragma unroll
  for (int i = 0; i < NR; ++i) S[i] = (live && s + i * NS < d) ? st[s + i * NS] : 0.f;
  const float A = expf(a_log[h]);
  const float qscale = rsqrtf((float)d);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  for (int t0 = 0; t0 < n; t0 += TC) {
    const int nt = n - t0 < TC ? n - t0 : TC;
    __syncthreads();  // the previous chunk has been read
    for (int t = warp; t < nt; t += n_warps) {
      const float* row = qkv + (size_t)(r0 + t0 + t) * ld;
      const float* qr = row + (size_t)kvh * d;
      const float* kr = row + (size_t)(G + kvh) * d;
      float qq = 0.f, kk = 0.f;
      for (int i = lane; i < d; i += 32) { qq = fmaf(qr[i], qr[i], qq); kk = fmaf(kr[i], kr[i], kk); }
      const float iq = qscale / sqrtf(warp_sum(qq) + 1e-6f), ik = 1.f / sqrtf(warp_sum(kk) + 1e-6f);
      const float* ar = a_raw + (size_t)(r0 + t0 + t) * H * d + (size_t)h * d;
      for (int i = lane; i < dp; i += 32) {
        const bool in = i < d;
        sq[(size_t)t * dp + i] = in ? qr[i] * iq : 0.f;
        sk[(size_t)t * dp + i] = in ? kr[i] * ik : 0.f;
        sg[(size_t)t * dp + i] = in ? expf(-A * softplusf_(ar[i] + dt_bias[(size_t)h * d + i])) : 1.f;
      }
      const float* vr = row + (size_t)2 * G * d + (size_t)h * dv + (size_t)blockIdx.z * PB;
      for (int i = lane; i < PB; i += 32) sv[(size_t)t * PB + i] = blockIdx.z * PB + i < dv ? vr[i] : 0.f;
      if (lane == 0) sb[t] = sigmoidf_(b_raw[(size_t)(r0 + t0 + t) * ld_b + b_col + h]);
    }
    __syncthreads();
    {  // every thread of a warp takes part (the sums shuffle across whole warps); spare threads work on zeros
      const int cv = col_local < PB ? col_local : PB - 1;
      for (int t = 0; t < nt; ++t) {
        const float* gq = sq + (size_t)t * dp + s;
        const float* gk = sk + (size_t)t * dp + s;
        const float* gg = sg + (size_t)t * dp + s;
        float part = 0.f;
#pragma unroll
        for (int i = 0; i < NR; ++i) {
          S[i] *= gg[i * NS];
          part = fmaf(S[i], gk[i * NS], part);
        }
        part = group_sum(part, NS);
        const float u = sb[t] * (sv[(size_t)t * PB + cv] - part);
        float po = 0.f;
#pragma unroll
        for (int i = 0; i < NR; ++i) {
          S[i] = fmaf(gk[i * NS], u, S[i]);
          po = fmaf(S[i], gq[i * NS], po);
        }
        po = group_sum(po, NS);
        if (s == 0 && live) out[(size_t)(r0 + t0 + t) * H * dv + (size_t)h * dv + col] = po;
      }
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NR; ++i)
      if (s + i * NS < d) st[s + i * NS] = S[i];
  }
}

// proj: 32-bit rows of stride ld: q heads at q_col (H heads of d), k at k_col, v at v_col (H heads of dv), the raw
// input gate of head h at i_col + h, the raw forget gate at f_col + h (their biases i_bias, f_bias are added here).
// mem: [slots, H, dv, d]; nrm: [slots, H, d]; mx: [slots, H]. out: [rows, H dv].
// The block's columns are its PB value columns and one more that carries n (its "value" is 1), so n . q comes out
// of the same loop; the division waits until the chunk's sums are in shared memory.
template <int NR>
__global__ void mlstm_scan_kernel(const float* __restrict__ proj, int ld, int q_col, int k_col, int v_col, int i_col,
                                  int f_col, const float* __restrict__ i_bias, const float* __restrict__ f_bias,
                                  float cap, float* __restrict__ mem, float* __restrict__ nrm, float* __restrict__ mx,
                                  float* __restrict__ out, const int* __restrict__ req_row0,
                                  const int* __restrict__ req_count, const int* __restrict__ slots, int H, int d,
                                  int dv, int NS, int PB, int TC) {
  extern __shared__ __align__(16) float sm[];
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.x, rq = blockIdx.y;
  const int slot = slots[rq], n = req_count[rq], r0 = req_row0[rq];
  if (slot < 0 || n <= 0) return;
  const int dp = NS * NR;
  float* sq = sm;                          // [TC][dp]
  float* sk = sq + (size_t)TC * dp;        // [TC][dp]
  float* sv = sk + (size_t)TC * dp;        // [TC][PB + 1]
  float* so = sv + (size_t)TC * (PB + 1);  // [TC][PB + 1]
  float* keep = so + (size_t)TC * (PB + 1);  // [TC] e^(f + m - m')
  float* take = keep + TC;                 // [TC] e^(i - m')
  float* floor_ = take + TC;               // [TC] e^(-m')
  const int col_local = threadIdx.x / NS, s = threadIdx.x % NS;
  const bool is_n = col_local == PB;
  const int col = blockIdx.z * PB + col_local;
  const bool live = is_n || (col_local < PB && col < dv);
  float S[NR];
  float* st = is_n ? nrm + ((size_t)slot * H + h) * d
                   : mem + (((size_t)slot * H + h) * dv + (col < dv ? col : 0)) * d;
#pragma unroll
  for (int i = 0; i < NR; ++i) S[i] = (live && col_local <= PB && s + i * NS < d) ? st[s + i * NS] : 0.f;
  float m = mx[(size_t)slot * H + h];  // thread 0 carries it
  const float qscale = rsqrtf((float)d);
  const float bi = i_bias ? i_bias[h] : 0.f, bf = f_bias ? f_bias[h] : 0.f;
  for (int t0 = 0; t0 < n; t0 += TC) {
    const int nt = n - t0 < TC ? n - t0 : TC;
    __syncthreads();
    for (int e = threadIdx.x; e < nt * dp; e += blockDim.x) {
      const int t = e / dp, i = e % dp;
      const float* row = proj + (size_t)(r0 + t0 + t) * ld;
      sq[e] = i < d ? row[q_col + (size_t)h * d + i] * qscale : 0.f;
      sk[e] = i < d ? row[k_col + (size_t)h * d + i] : 0.f;
    }
    for (int e = threadIdx.x; e < nt * (PB + 1); e += blockDim.x) {
      const int t = e / (PB + 1), i = e % (PB + 1);
      const float* row = proj + (size_t)(r0 + t0 + t) * ld;
      sv[e] = i == PB ? 1.f : (blockIdx.z * PB + i < dv ? row[v_col + (size_t)h * dv + blockIdx.z * PB + i] : 0.f);
    }
    if (threadIdx.x == 0) {
      for (int t = 0; t < nt; ++t) {
        const float* row = proj + (size_t)(r0 + t0 + t) * ld;
        const float gi = cap * tanhf((row[i_col + h] + bi) / cap);
        const float gf = log_sigmoidf_(cap * tanhf((row[f_col + h] + bf) / cap));
        const float m_new = fmaxf(gf + m, gi);
        keep[t] = expf(gf + m - m_new);
        take[t] = expf(gi - m_new);
        floor_[t] = expf(-m_new);
        m = m_new;
      }
    }
    __syncthreads();
    {  // every thread of a warp takes part (the sums shuffle across whole warps); spare threads work on zeros
      const int cv = col_local <= PB ? col_local : PB;
      for (int t = 0; t < nt; ++t) {
        const float* gq = sq + (size_t)t * dp + s;
        const float* gk = sk + (size_t)t * dp + s;
        const float kp = keep[t], w = take[t] * sv[(size_t)t * (PB + 1) + cv];
        float po = 0.f;
#pragma unroll
        for (int i = 0; i < NR; ++i) {
          S[i] = fmaf(kp, S[i], w * gk[i * NS]);
          po = fmaf(S[i], gq[i * NS], po);
        }
        po = group_sum(po, NS);
        if (s == 0 && col_local <= PB) so[(size_t)t * (PB + 1) + col_local] = po;
      }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < nt * PB; e += blockDim.x) {
      const int t = e / PB, i = e % PB;
      if (blockIdx.z * PB + i < dv) {
        const float den = fmaxf(fabsf(so[(size_t)t * (PB + 1) + PB]), floor_[t]) + 1e-6f;
        out[(size_t)(r0 + t0 + t) * H * dv + (size_t)h * dv + blockIdx.z * PB + i] = so[(size_t)t * (PB + 1) + i] / den;
      }
    }
  }
  if (live && col_local <= PB && (!is_n || blockIdx.z == 0)) {
#pragma unroll
    for (int i = 0; i < NR; ++i)
      if (s + i * NS < d) st[s + i * NS] = S[i];
  }
  if (threadIdx.x == 0 && blockIdx.z == 0) mx[(size_t)slot * H + h] = m;
}

// o: [rows, H dv] 32-bit. out[r, h, j] = o / sqrt(mean_j o^2 + eps) * w[h * w_head + j] * sigmoid(gate[r, h dv + j]);
// w_head 0: one weight vector for every head. gate: rows of stride ld_g (TG), null for none.
template <typename TG, typename TO>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, int w_head,
                      const TG* __restrict__ gate, int ld_g, TO* __restrict__ out, int H, int dv, float eps) {
  __shared__ float red[4];
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.x;
  const size_t row = blockIdx.y;
  const float* orow = o + (row * H + h) * dv;
  float ss = 0.f;
  for (int j = threadIdx.x; j < dv; j += 128) ss = fmaf(orow[j], orow[j], ss);
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  const float inv = 1.f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)dv + eps);
  for (int j = threadIdx.x; j < dv; j += 128) {
    float v = orow[j] * inv * w[(size_t)h * w_head + j];
    if (gate) v *= sigmoidf_(to_f32(gate[row * ld_g + (size_t)h * dv + j]));
    out[(row * H + h) * dv + j] = from_f32<TO>(v);
  }
}

// (threads per value column, state rows per thread) for d key channels
bool split_rows(int d, int* ns_out, int* nr_out) {
  int ns = 1;
  while ((d + ns - 1) / ns > MAXR && ns < 32) ns <<= 1;
  if ((d + ns - 1) / ns > MAXR) return false;
  while (ns < 8 && ns * 8 <= d) ns <<= 1;  // shorter chains per thread: at least eight rows each, up to eight threads
  *ns_out = ns;
  *nr_out = (d + ns - 1) / ns;
  return true;
}

int round_nr(int nr) { return nr <= 4 ? 4 : nr <= 8 ? 8 : nr <= 16 ? 16 : 32; }

}  // namespace

CUCA_API int cuca_matrix_state_max_dim() { return 32 * MAXR; }

CUCA_API int cuca_delta_scan(const float* qkv, int ld, const float* a_raw, const float* dt_bias, const float* a_log,
                             const float* b_raw, int ld_b, int b_col, float* state, float* out, const int* req_row0,
                             const int* req_count, const int* slots, int n_seqs, int H, int G, int d, int dv,
                             cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  CUCA_REQUIRE(H > 0 && G > 0 && H % G == 0 && d > 0 && dv > 0, "delta_scan: bad sizes heads=%d key heads=%d dim=%d vdim=%d",
               H, G, d, dv);
  CUCA_REQUIRE(n_seqs <= 65535, "delta_scan: %d requests exceed the launch limit", n_seqs);
  int ns, nr;
  CUCA_REQUIRE(split_rows(d, &ns, &nr), "delta_scan: %d key channels exceed %d", d, 32 * MAXR);
  nr = round_nr(nr);
  int pb = 128 / ns;
  pb = pb > dv ? dv : pb;
  const int threads = (pb * ns + 31) / 32 * 32;
  const int dp = ns * nr;
  int tc = 40960 / ((3 * dp + pb + 1) * 4);
  tc = tc > 16 ? 16 : tc;
  CUCA_REQUIRE(tc >= 1, "delta_scan: a token of %d key channels does not fit shared memory", d);
  const size_t smem = (size_t)tc * (3 * dp + pb + 1) * 4;
  dim3 grid(H, n_seqs, (dv + pb - 1) / pb);
#define DS(NR)                                                                                                    \
  cuca_launch(delta_scan_kernel<NR>, grid, dim3(threads), smem, stream, true, qkv, ld, a_raw, dt_bias, a_log, b_raw, \
              ld_b, b_col, state, out, req_row0, req_count, slots, H, G, d, dv, ns, pb, tc)
  if (nr == 4) DS(4);
  else if (nr == 8) DS(8);
  else if (nr == 16) DS(16);
  else DS(32);
#undef DS
  CUCA_CHECK_LAUNCH("delta_scan");
  return 0;
}

CUCA_API int cuca_mlstm_scan(const float* proj, int ld, int q_col, int k_col, int v_col, int i_col, int f_col,
                             const float* i_bias, const float* f_bias, float cap, float* mem, float* nrm, float* mx,
                             float* out, const int* req_row0, const int* req_count, const int* slots, int n_seqs,
                             int H, int d, int dv, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  CUCA_REQUIRE(H > 0 && d > 0 && dv > 0 && cap > 0.f, "mlstm_scan: bad sizes heads=%d dim=%d vdim=%d cap=%g", H, d, dv,
               (double)cap);
  CUCA_REQUIRE(n_seqs <= 65535, "mlstm_scan: %d requests exceed the launch limit", n_seqs);
  int ns, nr;
  CUCA_REQUIRE(split_rows(d, &ns, &nr), "mlstm_scan: %d key channels exceed %d", d, 32 * MAXR);
  nr = round_nr(nr);
  int pb = 128 / ns - 1;  // one more column carries n
  pb = pb < 1 ? 1 : (pb > dv ? dv : pb);
  const int threads = ((pb + 1) * ns + 31) / 32 * 32;
  const int dp = ns * nr;
  const int per = 2 * dp + 2 * (pb + 1) + 3;
  int tc = 40960 / (per * 4);
  tc = tc > 16 ? 16 : tc;
  CUCA_REQUIRE(tc >= 1, "mlstm_scan: a token of %d key channels does not fit shared memory", d);
  const size_t smem = (size_t)tc * per * 4;
  dim3 grid(H, n_seqs, (dv + pb - 1) / pb);
#define MS(NR)                                                                                                      \
  cuca_launch(mlstm_scan_kernel<NR>, grid, dim3(threads), smem, stream, true, proj, ld, q_col, k_col, v_col, i_col,   \
              f_col, i_bias, f_bias, cap, mem, nrm, mx, out, req_row0, req_count, slots, H, d, dv, ns, pb, tc)
  if (nr == 4) MS(4);
  else if (nr == 8) MS(8);
  else if (nr == 16) MS(16);
  else MS(32);
#undef MS
  CUCA_CHECK_LAUNCH("mlstm_scan");
  return 0;
}

CUCA_API int cuca_head_norm_gate(const float* o, const float* w, int w_head, const void* gate, int gate_dtype, int ld_g,
                                 void* out, int out_dtype, int n_rows, int H, int dv, float eps, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CUCA_REQUIRE(n_rows <= 65535, "head_norm_gate: %d rows exceed the launch limit", n_rows);
  dim3 grid(H, n_rows);
#define HNG(TG, TO)                                                                                              \
  cuca_launch(head_norm_gate_kernel<TG, TO>, grid, dim3(128), 0, stream, true, o, w, w_head, (const TG*)gate, ld_g, \
              (TO*)out, H, dv, eps)
  if (gate_dtype == CUCA_F32 && out_dtype == CUCA_F32) HNG(float, float);
  else if (gate_dtype == CUCA_F32 && out_dtype == CUCA_BF16) HNG(float, __nv_bfloat16);
  else if (gate_dtype == CUCA_BF16 && out_dtype == CUCA_BF16) HNG(__nv_bfloat16, __nv_bfloat16);
  else CUCA_REQUIRE(false, "head_norm_gate: unsupported dtypes %d/%d", gate_dtype, out_dtype);
#undef HNG
  CUCA_CHECK_LAUNCH("head_norm_gate");
  return 0;
}
