// Generalised delta rule with a matrix state per head, carried from token to token.
//
// Per token and head, key channel c and value channel d (D of each):
//     decay_c = exp(-exp(-1/2) * sigmoid(w0_c + sum_l W2[c,l] tanh(low_l)))
//     rate_c  = sigmoid(a_c + bias_c)
//     u       = k / sqrt(sum_c k_c^2 + 1e-6)
//     S[c,d] <- decay_c S[c,d] - rate_c u_c (sum_c' u_c' S[c',d]) + k_c v_d     (old S on the right)
//     o_d     = sum_c S[c,d] r_c
//     y       = o / sqrt(mean_d o_d^2 + eps) * gain * sigmoid(g)
// The projections r, k, v, g, a, low arrive as columns of one matrix product (activation
// dtype); everything after them is float32: decays, rates, the unit key, the state, the
// head-wise norm and the gate.  Three kernels:
//   prepare     per token, in parallel: decay, u, rate*u, and k, r, v widened, as float32
//   recurrence  per (sequence, head, slice of value channels): the scan over the step's
//               tokens; the state comes from and returns to the request's slot; the tokens'
//               inputs stream through a ring of shared-memory stages filled by cp.async
//   output      per token, in parallel: head-wise norm, gain, gate
// The scan's order is the token order, so a sequence's result is the same however its tokens
// were cut into steps and whatever else the batch holds.
#include "common.cuh"

namespace si {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

constexpr int DELTA_PLANES = 6;   // prep[t][plane][heads*D]: decay, u, rate*u, k, r, v

// proj columns: [r | k | v | g | a | low], each of the first five HD = heads*D wide, low L wide.
// w2t is the decay's second matrix transposed, [L, HD], so that neighbouring channels read
// neighbouring words.  A block takes TG tokens of one head: with many tokens (prompts) a word of
// w2t serves eight of them, with few (decoding) every token has blocks of its own.
template <typename T, int TG>
__global__ void delta_prepare_kernel(const T* __restrict__ proj, int proj_stride,
                                     const T* __restrict__ w2t, const float* __restrict__ w0,
                                     const float* __restrict__ a_bias, float* __restrict__ prep,
                                     int n_tokens, int heads, int D, int L) {
  extern __shared__ float low_s[];             // [TG][L] tanh of the inner projection
  __shared__ float part[TG][32];               // per token: the warps' sums of k^2
  const int t0 = blockIdx.x * TG, h = blockIdx.y, c = threadIdx.x;
  const int nt = min(TG, n_tokens - t0);
  const int HD = heads * D;
  const bool mine = c < D;
  const int col = h * D + c;
  const int lane = c & 31, warp = c >> 5, n_warps = (blockDim.x + 31) >> 5;
  // weights first: no kernel of the step writes them
  const float bias = mine ? a_bias[col] : 0.0f;
  const float z0 = mine ? w0[col] : 0.0f;
  pdl_wait();
  pdl_trigger();
  for (int idx = threadIdx.x; idx < TG * L; idx += blockDim.x) {
    const int tt = idx / L, l = idx - tt * L;
    low_s[idx] = tt < nt ? tanhf(to_f32<T>(proj[(size_t)(t0 + tt) * proj_stride + 5 * HD + l])) : 0.0f;
  }
  float k[TG], r_in[TG], v_in[TG], a_in[TG];
#pragma unroll
  for (int tt = 0; tt < TG; ++tt) {
    const bool on = mine && tt < nt;
    const T* row = proj + (size_t)(t0 + (tt < nt ? tt : 0)) * proj_stride;
    k[tt] = on ? to_f32<T>(row[HD + col]) : 0.0f;
    r_in[tt] = on ? to_f32<T>(row[col]) : 0.0f;
    v_in[tt] = on ? to_f32<T>(row[2 * HD + col]) : 0.0f;
    a_in[tt] = on ? to_f32<T>(row[4 * HD + col]) : 0.0f;
  }
#pragma unroll
  for (int tt = 0; tt < TG; ++tt) {
    const float sq = warp_sum(k[tt] * k[tt]);
    if (lane == 0) part[tt][warp] = sq;
  }
  __syncthreads();   // low_s and part are complete
  if (!mine) return;
  float z[TG];
#pragma unroll
  for (int tt = 0; tt < TG; ++tt) z[tt] = z0;
  // z = z0 + sum_l W2[c,l] low_l: term l goes to running sum l mod 4, the four are joined as
  // (0+1)+(2+3), whatever the number of tokens a block takes, so a token's decay does not depend
  // on whether it came alone (decoding) or in a prompt
  float zz[TG][4];
#pragma unroll
  for (int tt = 0; tt < TG; ++tt) zz[tt][0] = zz[tt][1] = zz[tt][2] = zz[tt][3] = 0.0f;
  int l = 0;
  auto four = [&]() {   // terms l .. l+3 of every token
    float w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) w[j] = to_f32<T>(w2t[(size_t)(l + j) * HD + col]);
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int tt = 0; tt < TG; ++tt) zz[tt][j] = __fmaf_rn(w[j], low_s[tt * L + l + j], zz[tt][j]);
  };
  if (TG == 1) {
    // one token: the block's time is the trips to memory for the decay matrix's words, so
    // thirty-two of them are asked for at once
#pragma unroll 8
    for (; l + 4 <= L; l += 4) four();
  } else {
#pragma unroll 2
    for (; l + 4 <= L; l += 4) four();
  }
  for (int j = 0; l < L; ++l, ++j) {   // up to three left over: they are terms 0, 1, 2 mod 4
    const float w = to_f32<T>(w2t[(size_t)l * HD + col]);
#pragma unroll
    for (int tt = 0; tt < TG; ++tt) {
      const float x = low_s[tt * L + l];   // explicit fused operations: the same in every instantiation
      if (j == 0) zz[tt][0] = __fmaf_rn(w, x, zz[tt][0]);
      else if (j == 1) zz[tt][1] = __fmaf_rn(w, x, zz[tt][1]);
      else zz[tt][2] = __fmaf_rn(w, x, zz[tt][2]);
    }
  }
#pragma unroll
  for (int tt = 0; tt < TG; ++tt)
    z[tt] = __fadd_rn(z[tt], __fadd_rn(__fadd_rn(zz[tt][0], zz[tt][1]), __fadd_rn(zz[tt][2], zz[tt][3])));
#pragma unroll
  for (int tt = 0; tt < TG; ++tt) {
    if (tt < nt) {
      float ss = 0.0f;
      for (int w = 0; w < n_warps; ++w) ss += part[tt][w];   // fixed order
      const float decay = expf(-0.60653065971263342f * sigmoidf_(z[tt]));
      const float u = k[tt] / sqrtf(ss + 1e-6f);
      const float rate = sigmoidf_(a_in[tt] + bias);
      float* dst = prep + (size_t)(t0 + tt) * DELTA_PLANES * HD + col;
      dst[0] = decay;
      dst[HD] = u;
      dst[2 * HD] = rate * u;
      dst[3 * HD] = k[tt];
      dst[4 * HD] = r_in[tt];
      dst[5 * HD] = v_in[tt];
    }
  }
}

// Threads of a block: DC value channels x KS lanes; lane ks of channel d keeps S[c][d] for
// c = ks*R + i, i < R, in registers (c >= D padded with zeros).  Tokens are taken in groups
// of TB; a group's inputs ([TB][5] key-side planes and [TB][DC] values) are one stage of a
// ring of NS stages that cp.async fills NS-1 groups ahead of the arithmetic.  In a plane each
// lane's R channels are followed by four unused words, so that the lanes' 16-byte reads fall
// into different banks.
constexpr int DELTA_DC = 32;   // value channels per block
constexpr int DELTA_TB = 8;    // tokens per stage
constexpr int DELTA_NS = 4;    // stages

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int R, int KS>
struct DeltaShape {
  static constexpr int PLANE = KS * (R + 4);                       // words of one plane of one token
  static constexpr int STAGE = DELTA_TB * (5 * PLANE + DELTA_DC);  // words of a stage
  __host__ __device__ static constexpr int at(int c) { return (c / R) * (R + 4) + (c % R); }
};

template <int R, int KS, bool VEC>
__global__ void __launch_bounds__(KS * DELTA_DC)
delta_recurrence_kernel(const float* __restrict__ prep, const int* __restrict__ cu_q,
                        const int* __restrict__ seq_slots, float* __restrict__ state,
                        float* __restrict__ o_out, int heads, int D) {
  extern __shared__ __align__(16) float sm[];
  using Sh = DeltaShape<R, KS>;
  constexpr int PLANE = Sh::PLANE, STAGE = Sh::STAGE, V_AT = DELTA_TB * 5 * PLANE;
  const int s = blockIdx.x, h = blockIdx.y;
  const int d0 = blockIdx.z * DELTA_DC;
  const int tid = threadIdx.x;
  const int ks = tid % KS, dl = tid / KS;
  const int d = d0 + dl;
  const bool col_ok = d < D;
  const int HD = heads * D;
  const int dc = min(DELTA_DC, D - d0);                  // value channels of this block
  const int t_begin = cu_q[s], t_end = cu_q[s + 1];     // the step's description: on the device
  const int slot = seq_slots[s];                        // before the step's first kernel
  // channels past D (and value channels past the head's) stay zero in every stage
  for (int i = tid; i < DELTA_NS * STAGE; i += blockDim.x) sm[i] = 0.0f;
  // what this thread copies for every token (16-byte runs): found once
  constexpr int NF = 2;
  int f_src[NF], f_dst[NF], f_step[NF];
  if (VEC) {
    const int per_plane = D / 4, per_tok = 5 * per_plane + (dc + 3) / 4;
#pragma unroll
    for (int n = 0; n < NF; ++n) {
      const int e = tid + n * (int)blockDim.x;
      f_src[n] = -1; f_dst[n] = 0; f_step[n] = 0;
      if (e < 5 * per_plane) {
        const int which = e / per_plane, c4 = (e - which * per_plane) * 4;
        f_src[n] = which * HD + c4;
        f_dst[n] = which * PLANE + Sh::at(c4);
        f_step[n] = 5 * PLANE;
      } else if (e < per_tok) {
        const int c4 = (e - 5 * per_plane) * 4;
        f_src[n] = 5 * HD + d0 + c4;
        f_dst[n] = V_AT + c4;
        f_step[n] = DELTA_DC;
      }
    }
  }
  __syncthreads();
  pdl_wait();
  pdl_trigger();
  float* S_g = state + ((size_t)slot * heads + h) * D * D;
  float S[R];   // lane ks owns the key channels ks*R .. ks*R + R - 1 of its column
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int c = ks * R + i;
    S[i] = (col_ok && c < D) ? S_g[(size_t)c * D + d] : 0.0f;
  }
  const int n_groups = (t_end - t_begin + DELTA_TB - 1) / DELTA_TB;
  auto fetch = [&](int g) {   // group g of the sequence into stage g % NS
    if (g < n_groups) {
      float* st = sm + (g % DELTA_NS) * STAGE;
      const int tb = t_begin + g * DELTA_TB;
      const int nt = min(DELTA_TB, t_end - tb);
      if (VEC) {   // D is a multiple of 4: every run starts on a 16-byte boundary
        const float* src = prep + (size_t)tb * DELTA_PLANES * HD + h * D;
#pragma unroll
        for (int n = 0; n < NF; ++n)
          if (f_src[n] >= 0)
            for (int tt = 0; tt < nt; ++tt)
              cp_async16(st + f_dst[n] + tt * f_step[n],
                         src + (size_t)tt * DELTA_PLANES * HD + f_src[n]);
      } else {
        const int per_tok = 5 * D + dc;
        for (int idx = tid; idx < nt * per_tok; idx += blockDim.x) {
          const int tt = idx / per_tok, e = idx - tt * per_tok;
          const float* src = prep + (size_t)(tb + tt) * DELTA_PLANES * HD + h * D;
          if (e < 5 * D) {
            const int which = e / D, c = e - which * D;
            cp_async4(st + (tt * 5 + which) * PLANE + Sh::at(c), src + (size_t)which * HD + c);
          } else {
            const int c = e - 5 * D;
            cp_async4(st + V_AT + tt * DELTA_DC + c, src + (size_t)5 * HD + d0 + c);
          }
        }
      }
    }
    cp_async_commit();   // an empty group keeps the count uniform
  };

  // One token: in[p] holds this lane's R channels of plane p (decay, u, rate*u, k, r).  Four
  // running sums keep the chains of dependent additions short; the order of the additions is
  // fixed, so the result does not depend on where the token sits in a step.
  constexpr int R4 = R / 4;
  auto token = [&](const float4 (&in)[5][R4], float v, int t) {
    float us[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int j = 0; j < R4; ++j) {
      us[0] = fmaf(in[1][j].x, S[4 * j], us[0]);
      us[1] = fmaf(in[1][j].y, S[4 * j + 1], us[1]);
      us[2] = fmaf(in[1][j].z, S[4 * j + 2], us[2]);
      us[3] = fmaf(in[1][j].w, S[4 * j + 3], us[3]);
    }
    float ust = (us[0] + us[1]) + (us[2] + us[3]);
#pragma unroll
    for (int o = KS / 2; o > 0; o >>= 1) ust += __shfl_xor_sync(0xffffffffu, ust, o);
    float os[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int j = 0; j < R4; ++j) {
      S[4 * j] = fmaf(in[0][j].x, S[4 * j], fmaf(in[3][j].x, v, -in[2][j].x * ust));
      S[4 * j + 1] = fmaf(in[0][j].y, S[4 * j + 1], fmaf(in[3][j].y, v, -in[2][j].y * ust));
      S[4 * j + 2] = fmaf(in[0][j].z, S[4 * j + 2], fmaf(in[3][j].z, v, -in[2][j].z * ust));
      S[4 * j + 3] = fmaf(in[0][j].w, S[4 * j + 3], fmaf(in[3][j].w, v, -in[2][j].w * ust));
      os[0] = fmaf(S[4 * j], in[4][j].x, os[0]);
      os[1] = fmaf(S[4 * j + 1], in[4][j].y, os[1]);
      os[2] = fmaf(S[4 * j + 2], in[4][j].z, os[2]);
      os[3] = fmaf(S[4 * j + 3], in[4][j].w, os[3]);
    }
    float ot = (os[0] + os[1]) + (os[2] + os[3]);
#pragma unroll
    for (int off = KS / 2; off > 0; off >>= 1) ot += __shfl_xor_sync(0xffffffffu, ot, off);
    if (ks == 0 && col_ok) o_out[(size_t)t * HD + h * D + d] = ot;
  };
  auto read = [&](float4 (&in)[5][R4], const float* st, int tt) {
    const float4* base = reinterpret_cast<const float4*>(st + tt * 5 * PLANE + ks * (R + 4));
#pragma unroll
    for (int pl = 0; pl < 5; ++pl)
#pragma unroll
      for (int j = 0; j < R4; ++j) in[pl][j] = base[pl * (PLANE / 4) + j];
  };

#pragma unroll
  for (int g = 0; g < DELTA_NS - 1; ++g) fetch(g);
  for (int g = 0; g < n_groups; ++g) {
    fetch(g + DELTA_NS - 1);          // into the stage that group g-1 has left
    cp_async_wait<DELTA_NS - 1>();    // this thread's copies of group g have landed
    __syncthreads();                  // and everyone else's
    const float* st = sm + (g % DELTA_NS) * STAGE;
    const float* v_s = st + V_AT;
    const int tb = t_begin + g * DELTA_TB;
    const int nt = min(DELTA_TB, t_end - tb);
    if (R <= 16) {
      // two sets of registers: the next token's inputs leave shared memory while this
      // token's sums run
      float4 a[5][R4], b[5][R4];
      read(a, st, 0);
      for (int tt = 0; tt < nt; tt += 2) {
        if (tt + 1 < nt) read(b, st, tt + 1);
        token(a, v_s[tt * DELTA_DC + dl], tb + tt);
        if (tt + 1 < nt) {
          if (tt + 2 < nt) read(a, st, tt + 2);
          token(b, v_s[(tt + 1) * DELTA_DC + dl], tb + tt + 1);
        }
      }
    } else {
      float4 a[5][R4];
      for (int tt = 0; tt < nt; ++tt) {
        read(a, st, tt);
        token(a, v_s[tt * DELTA_DC + dl], tb + tt);
      }
    }
    __syncthreads();   // the stage may be refilled
  }
  cp_async_wait<0>();
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int c = ks * R + i;
    if (col_ok && c < D) S_g[(size_t)c * D + d] = S[i];
  }
}

// A block per token and eight heads, a warp per head: the head's mean square over its D channels
// is a sum within the warp, in a fixed order.
constexpr int DELTA_OUT_WARPS = 8;

template <typename T, typename TW>
__global__ void __launch_bounds__(32 * DELTA_OUT_WARPS)
delta_output_kernel(const float* __restrict__ o, const T* __restrict__ proj, int proj_stride,
                    const TW* __restrict__ gain, T* __restrict__ out, int heads, int D, float eps) {
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int HD = heads * D;
  pdl_wait();
  pdl_trigger();
  const float* orow = o + (size_t)t * HD;
  const T* grow = proj + (size_t)t * proj_stride + 3 * HD;
  T* yrow = out + (size_t)t * HD;
  const int h = blockIdx.y * DELTA_OUT_WARPS + warp;
  if (h < heads) {
    float ss = 0.0f;
    for (int c = lane; c < D; c += 32) {
      const float x = orow[h * D + c];
      ss = fmaf(x, x, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)D + eps);
    for (int c = lane; c < D; c += 32) {
      const int col = h * D + c;
      const float g = sigmoidf_(to_f32<T>(grow[col]));
      yrow[col] = from_f32<T>(orow[col] * inv * to_f32<TW>(gain[col]) * g);
    }
  }
}

}  // namespace si

template <typename T, int TG>
static int launch_delta_prepare(const void* proj, int proj_stride, const void* w2t, const float* w0,
                                const float* a_bias, float* prep, int n_tokens, int heads, int D,
                                int L, cudaStream_t stream) {
  const int threads = (D + 31) / 32 * 32;
  dim3 grid((n_tokens + TG - 1) / TG, heads);
  const size_t smem = (size_t)TG * L * sizeof(float);
  if (smem > 48 * 1024) return SI_ERR_TOO_LARGE;
  SI_LAUNCH((si::delta_prepare_kernel<T, TG>), grid, threads, smem, stream, (const T*)proj, proj_stride,
            (const T*)w2t, w0, a_bias, prep, n_tokens, heads, D, L);
  return SI_OK;
}

SI_API int si_delta_prepare(const void* proj, int proj_stride, const void* w2t, const float* w0,
                            const float* a_bias, float* prep, int n_tokens, int heads, int D, int L,
                            int dtype, cudaStream_t stream) {
  if (!proj || !w2t || !w0 || !a_bias || !prep || n_tokens < 0 || heads <= 0 || D <= 0 || L <= 0)
    return SI_ERR_ARG;
  if (D > 1024 || heads > 65535) return SI_ERR_TOO_LARGE;
  if (n_tokens == 0) return SI_OK;
  const bool many = n_tokens >= 64;
  if (dtype == SI_BF16)
    return many ? launch_delta_prepare<__nv_bfloat16, 8>(proj, proj_stride, w2t, w0, a_bias, prep,
                                                         n_tokens, heads, D, L, stream)
                : launch_delta_prepare<__nv_bfloat16, 1>(proj, proj_stride, w2t, w0, a_bias, prep,
                                                         n_tokens, heads, D, L, stream);
  if (dtype == SI_F32)
    return many ? launch_delta_prepare<float, 8>(proj, proj_stride, w2t, w0, a_bias, prep, n_tokens,
                                                 heads, D, L, stream)
                : launch_delta_prepare<float, 1>(proj, proj_stride, w2t, w0, a_bias, prep, n_tokens,
                                                 heads, D, L, stream);
  return SI_ERR_DTYPE;
}

template <int R, int KS, bool VEC>
static int launch_delta_recurrence(const float* prep, const int* cu_q, const int* seq_slots,
                                   float* state, float* o_out, int n_seqs, int heads, int D,
                                   cudaStream_t stream) {
  const size_t smem = (size_t)si::DELTA_NS * si::DeltaShape<R, KS>::STAGE * sizeof(float);
  auto kern = si::delta_recurrence_kernel<R, KS, VEC>;
  if (smem > 48 * 1024) SI_ALLOW_DYNAMIC_SMEM(kern, smem);
  dim3 grid(n_seqs, heads, (D + si::DELTA_DC - 1) / si::DELTA_DC);
  SI_LAUNCH(kern, grid, KS * si::DELTA_DC, smem, stream, prep, cu_q, seq_slots, state, o_out, heads, D);
  return SI_OK;
}

// state: [slots, heads, D, D] float32 (key channel, value channel); sequence s of the step owns
// the tokens cu_q[s]..cu_q[s+1]-1 and the slot seq_slots[s].  prep: what si_delta_prepare
// wrote.  o_out: [n_tokens, heads*D] float32.  Heads of 32 channels and more spread a column's
// key channels over eight lanes, smaller ones over four.
SI_API int si_delta_recurrence(const float* prep, const int* cu_q, const int* seq_slots,
                               float* state, float* o_out, int n_seqs, int heads, int D,
                               cudaStream_t stream) {
  if (!prep || !cu_q || !seq_slots || !state || !o_out || n_seqs < 0 || heads <= 0 || D <= 0)
    return SI_ERR_ARG;
  if (heads > 65535) return SI_ERR_TOO_LARGE;
  if (n_seqs == 0) return SI_OK;
#define SI_DELTA_CASE(R, KS)                                                                       \
  if (D <= R * KS)                                                                                 \
    return D % 4 == 0 ? launch_delta_recurrence<R, KS, true>(prep, cu_q, seq_slots, state, o_out,  \
                                                             n_seqs, heads, D, stream)             \
                      : launch_delta_recurrence<R, KS, false>(prep, cu_q, seq_slots, state, o_out, \
                                                              n_seqs, heads, D, stream);
  SI_DELTA_CASE(4, 4)
  SI_DELTA_CASE(4, 8)
  SI_DELTA_CASE(8, 8)
  SI_DELTA_CASE(16, 8)
  SI_DELTA_CASE(32, 8)
#undef SI_DELTA_CASE
  return SI_ERR_UNSUPPORTED;  // heads of more than 256 channels
}

SI_API int si_delta_output(const float* o, const void* proj, int proj_stride, const void* gain,
                           void* out, int n_tokens, int heads, int D, float eps, int dtype,
                           int gain_dtype, cudaStream_t stream) {
  if (!o || !proj || !gain || !out || n_tokens < 0 || heads <= 0 || D <= 0 || !(eps > 0.0f))
    return SI_ERR_ARG;
  if (n_tokens == 0) return SI_OK;
  const int threads = 32 * si::DELTA_OUT_WARPS;
  if (heads > 65535 * si::DELTA_OUT_WARPS) return SI_ERR_TOO_LARGE;
  const dim3 grid(n_tokens, (heads + si::DELTA_OUT_WARPS - 1) / si::DELTA_OUT_WARPS);
  if (dtype == SI_BF16 && gain_dtype == SI_BF16)
    SI_LAUNCH((si::delta_output_kernel<__nv_bfloat16, __nv_bfloat16>), grid, threads, 0, stream, o,
              (const __nv_bfloat16*)proj, proj_stride, (const __nv_bfloat16*)gain, (__nv_bfloat16*)out,
              heads, D, eps);
  else if (dtype == SI_BF16 && gain_dtype == SI_F32)
    SI_LAUNCH((si::delta_output_kernel<__nv_bfloat16, float>), grid, threads, 0, stream, o,
              (const __nv_bfloat16*)proj, proj_stride, (const float*)gain, (__nv_bfloat16*)out, heads,
              D, eps);
  else if (dtype == SI_F32 && gain_dtype == SI_F32)
    SI_LAUNCH((si::delta_output_kernel<float, float>), grid, threads, 0, stream, o,
              (const float*)proj, proj_stride, (const float*)gain, (float*)out, heads, D, eps);
  else
    return SI_ERR_DTYPE;
  return SI_OK;
}
