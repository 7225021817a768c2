// Recurrent mixers for ragged token batches: the generalised delta rule with a per-channel decay.
//
// Per head, with a state S [dim x dim] (key channel i, value column j) kept in fp32 per sequence slot:
//     u   = k / sqrt(sum(k^2) + key_eps)
//     S  <- diag(w) S - (a * u) (u^T S) + k v^T          (both first terms read the old S)
//     o   = S^T r
// Everything that enters the recurrence besides the projections themselves is fp32: the decay w, the removal rate a,
// the unit key u, the state and the output.
//
// delta_prep_kernel   (CTA per token)   : w = exp(-decay_scale * sigmoid(W2 tanh(lora) + w0)), a = sigmoid(a_pre + a_bias),
//                                         u; writes w, u and a * u as fp32 rows.
// delta_rule_kernel   (warp per (sequence segment, head, 32 value columns)): a lane owns one value column of the state
//                                         in registers; the u^T S and S^T r products are then per-lane dot products
//                                         with vectors that all lanes read from shared memory, so the tokens of a
//                                         segment need no cross-lane traffic at all.  Token inputs are staged in
//                                         chunks.  The state is loaded from / stored to the slot's state once per
//                                         launch, which makes a prompt portion and a single decoded token the same case.
// headnorm_gate_kernel (warp per (token, head)): o / rms(o) per head, times a weight, times sigmoid(gate), times a
//                                         constant, rounded to the model dtype as the output projection's operand.
#include "common.cuh"

namespace pg {

__device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); }

template <typename T>
__global__ void delta_prep_kernel(float* __restrict__ decay, float* __restrict__ unit, float* __restrict__ rem,
                                  const T* __restrict__ proj, int ld, int k_col0, int a_col0, int lora_col0, int lora,
                                  const T* __restrict__ w2, const T* __restrict__ w0, const T* __restrict__ a_bias,
                                  int heads, int dim, float decay_scale, float key_eps) {
  extern __shared__ float sm[];           // [lora] tanh of the decay's inner projection | [heads] sum of k^2
  float* lo = sm;
  float* ksq = sm + lora;
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, nd = heads * dim;
  const T* row = proj + (size_t)t * ld;
  for (int j = threadIdx.x; j < lora; j += blockDim.x) lo[j] = tanhf(to_f<T>(row[lora_col0 + j]));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int h = warp; h < heads; h += warps) {
    float s = 0.f;
    for (int c = lane; c < dim; c += 32) { const float v = to_f<T>(row[k_col0 + h * dim + c]); s += v * v; }
    s = warp_sum(s);
    if (lane == 0) ksq[h] = s;
  }
  __syncthreads();
  for (int c = threadIdx.x; c < nd; c += blockDim.x) {
    float z = to_f<T>(w0[c]);
    const T* wr = w2 + (size_t)c * lora;
    for (int j = 0; j < lora; ++j) z = fmaf(to_f<T>(wr[j]), lo[j], z);
    const float w = expf(-decay_scale * sigmoid_f(z));
    float a = to_f<T>(row[a_col0 + c]);
    if (a_bias) a += to_f<T>(a_bias[c]);
    a = sigmoid_f(a);
    const float u = to_f<T>(row[k_col0 + c]) / sqrtf(ksq[c / dim] + key_eps);
    const size_t o = (size_t)t * nd + c;
    decay[o] = w;
    unit[o] = u;
    rem[o] = a * u;
  }
}

// segs: [n_segs][3] = {state slot, first token row, tokens}; the tokens of a segment are consecutive rows of one
// sequence in position order.  A segment with 0 tokens is skipped (the list is padded to a fixed length so that a
// captured launch stays valid).
template <typename T, int DMAX, int CH>
__global__ void __launch_bounds__(32)
delta_rule_kernel(float* __restrict__ out, float* __restrict__ state, const T* __restrict__ proj, int ld, int r_col0,
                  int k_col0, int v_col0, const float* __restrict__ decay, const float* __restrict__ unit,
                  const float* __restrict__ rem, const int32_t* __restrict__ segs, int heads, int dim) {
  __shared__ __align__(16) float sh[CH][5][DMAX];   // r, k, w, u, a*u of CH tokens
  __shared__ float sv[CH][32];                      // this warp's 32 value columns
  pdl_launch_dependents();
  pdl_wait();
  const int32_t* sg = segs + 3 * (size_t)blockIdx.x;
  const int slot = sg[0], row0 = sg[1], n = sg[2];
  if (n <= 0) return;
  const int h = blockIdx.y, lane = threadIdx.x, j = blockIdx.z * 32 + lane, nd = heads * dim;
  const bool live = j < dim;
  float S[DMAX];
  float* st = state + ((size_t)slot * heads + h) * dim * dim;
#pragma unroll
  for (int i = 0; i < DMAX; ++i) S[i] = (live && i < dim) ? st[(size_t)i * dim + j] : 0.f;
  for (int t0 = 0; t0 < n; t0 += CH) {
    const int nt = min(CH, n - t0);
    __syncwarp();
    for (int idx = lane; idx < nt * DMAX; idx += 32) {
      const int tt = idx / DMAX, c = idx % DMAX;
      const size_t trow = (size_t)row0 + t0 + tt;
      const bool in = c < dim;
      const size_t o = trow * nd + h * dim + c;
      sh[tt][0][c] = in ? to_f<T>(proj[trow * ld + r_col0 + h * dim + c]) : 0.f;
      sh[tt][1][c] = in ? to_f<T>(proj[trow * ld + k_col0 + h * dim + c]) : 0.f;
      sh[tt][2][c] = in ? decay[o] : 0.f;
      sh[tt][3][c] = in ? unit[o] : 0.f;
      sh[tt][4][c] = in ? rem[o] : 0.f;
    }
    for (int tt = 0; tt < nt; ++tt)
      sv[tt][lane] = live ? to_f<T>(proj[((size_t)row0 + t0 + tt) * ld + v_col0 + h * dim + j]) : 0.f;
    __syncwarp();
    for (int tt = 0; tt < nt; ++tt) {
      const float vj = sv[tt][lane];
      float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;            // u^T S over this lane's column
#pragma unroll
      for (int i = 0; i < DMAX; i += 4) {
        const float4 u4 = *reinterpret_cast<const float4*>(&sh[tt][3][i]);
        d0 = fmaf(u4.x, S[i], d0); d1 = fmaf(u4.y, S[i + 1], d1); d2 = fmaf(u4.z, S[i + 2], d2); d3 = fmaf(u4.w, S[i + 3], d3);
      }
      const float us = (d0 + d1) + (d2 + d3);
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
      for (int i = 0; i < DMAX; i += 4) {
        const float4 w4 = *reinterpret_cast<const float4*>(&sh[tt][2][i]);
        const float4 a4 = *reinterpret_cast<const float4*>(&sh[tt][4][i]);
        const float4 k4 = *reinterpret_cast<const float4*>(&sh[tt][1][i]);
        const float4 r4 = *reinterpret_cast<const float4*>(&sh[tt][0][i]);
        S[i] = fmaf(k4.x, vj, fmaf(-a4.x, us, w4.x * S[i]));
        S[i + 1] = fmaf(k4.y, vj, fmaf(-a4.y, us, w4.y * S[i + 1]));
        S[i + 2] = fmaf(k4.z, vj, fmaf(-a4.z, us, w4.z * S[i + 2]));
        S[i + 3] = fmaf(k4.w, vj, fmaf(-a4.w, us, w4.w * S[i + 3]));
        o0 = fmaf(r4.x, S[i], o0); o1 = fmaf(r4.y, S[i + 1], o1); o2 = fmaf(r4.z, S[i + 2], o2); o3 = fmaf(r4.w, S[i + 3], o3);
      }
      if (live) out[((size_t)row0 + t0 + tt) * nd + h * dim + j] = (o0 + o1) + (o2 + o3);
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < DMAX; ++i)
      if (i < dim) st[(size_t)i * dim + j] = S[i];
  }
}

template <typename T>
__global__ void headnorm_gate_kernel(T* __restrict__ out, int ld_out, const float* __restrict__ o, const T* __restrict__ w,
                                     const T* __restrict__ gate, int ld_gate, int n_tokens, int heads, int dim, float eps,
                                     float out_scale) {
  pdl_launch_dependents();
  pdl_wait();
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= (long long)n_tokens * heads) return;
  const int t = (int)(item / heads), h = (int)(item % heads);
  const float* orow = o + ((size_t)t * heads + h) * dim;
  float ss = 0.f;
  for (int c = lane; c < dim; c += 32) ss += orow[c] * orow[c];
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)dim + eps);
  for (int c = lane; c < dim; c += 32) {
    float v = orow[c] * inv;
    if (w) v *= to_f<T>(w[h * dim + c]);
    if (gate) v *= sigmoid_f(to_f<T>(gate[(size_t)t * ld_gate + h * dim + c]));
    out[(size_t)t * ld_out + h * dim + c] = from_f<T>(v * out_scale);
  }
}

template <typename T, int DMAX, int CH>
static int launch_delta(float* out, float* state, const void* proj, int ld, int r_col0, int k_col0, int v_col0,
                        const float* decay, const float* unit, const float* rem, const int32_t* segs, int n_segs,
                        int heads, int dim, cudaStream_t st) {
  return launch_pdl("delta_rule", delta_rule_kernel<T, DMAX, CH>, dim3(n_segs, heads, cdiv(dim, 32)), dim3(32), 0, st, out,
                    state, (const T*)proj, ld, r_col0, k_col0, v_col0, decay, unit, rem, segs, heads, dim);
}

}  // namespace pg

using namespace pg;

extern "C" int pg_delta_prep(float* decay, float* unit, float* rem, const void* proj, int ld, int k_col0, int a_col0,
                             int lora_col0, int lora, const void* w2, const void* w0, const void* a_bias, int n_tokens,
                             int heads, int dim, float decay_scale, float key_eps, int dtype, void* stream) {
  if (n_tokens <= 0) return PG_OK;
  PG_REQUIRE(decay && unit && rem && proj && w2 && w0 && lora > 0 && heads > 0 && dim > 0, "delta_prep: bad arguments");
  const size_t smem = sizeof(float) * ((size_t)lora + heads);
  PG_DISPATCH_DTYPE(dtype, T, {
    return launch_pdl("delta_prep", delta_prep_kernel<T>, dim3(n_tokens), dim3(heads * dim >= 1024 ? 256 : 128), smem,
                      (cudaStream_t)stream, decay, unit, rem, (const T*)proj, ld, k_col0, a_col0, lora_col0, lora,
                      (const T*)w2, (const T*)w0, (const T*)a_bias, heads, dim, decay_scale, key_eps);
  });
  return PG_OK;
}

extern "C" int pg_delta_rule(float* out, float* state, const void* proj, int ld, int r_col0, int k_col0, int v_col0,
                             const float* decay, const float* unit, const float* rem, const int32_t* segs, int n_segs,
                             int heads, int dim, int dtype, void* stream) {
  if (n_segs <= 0) return PG_OK;
  PG_REQUIRE(out && state && proj && decay && unit && rem && segs, "delta_rule: bad arguments");
  PG_REQUIRE(dim > 0 && dim <= 256, "delta_rule: head size %d (1..256)", dim);
  cudaStream_t st = (cudaStream_t)stream;
  PG_DISPATCH_DTYPE(dtype, T, {
    if (dim <= 32) return launch_delta<T, 32, 8>(out, state, proj, ld, r_col0, k_col0, v_col0, decay, unit, rem, segs, n_segs, heads, dim, st);
    if (dim <= 64) return launch_delta<T, 64, 8>(out, state, proj, ld, r_col0, k_col0, v_col0, decay, unit, rem, segs, n_segs, heads, dim, st);
    if (dim <= 128) return launch_delta<T, 128, 8>(out, state, proj, ld, r_col0, k_col0, v_col0, decay, unit, rem, segs, n_segs, heads, dim, st);
    return launch_delta<T, 256, 4>(out, state, proj, ld, r_col0, k_col0, v_col0, decay, unit, rem, segs, n_segs, heads, dim, st);
  });
  return PG_OK;
}

extern "C" int pg_headnorm_gate(void* out, int ld_out, const float* o, const void* w, const void* gate, int ld_gate,
                                int n_tokens, int heads, int dim, float eps, float out_scale, int dtype, void* stream) {
  if (n_tokens <= 0) return PG_OK;
  PG_REQUIRE(out && o && heads > 0 && dim > 0, "headnorm_gate: bad arguments");
  const int warps = 8;
  PG_DISPATCH_DTYPE(dtype, T, {
    return launch_pdl("headnorm_gate", headnorm_gate_kernel<T>, dim3(cdiv((long long)n_tokens * heads, warps)),
                      dim3(warps * 32), 0, (cudaStream_t)stream, (T*)out, ld_out, o, (const T*)w, (const T*)gate, ld_gate,
                      n_tokens, heads, dim, eps, out_scale);
  });
  return PG_OK;
}
