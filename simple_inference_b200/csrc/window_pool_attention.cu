// Grouped-query attention over a sliding window with pooled blocks before it, keys and values
// of different widths, a norm over the whole query and key projections, partial rotary
// positions and rotated values.  Generic kernels: any sizes, float32 or bfloat16 storage, all
// arithmetic in float32.  They are the attention of the 32-bit path and the yardstick of the
// tensor-core kernels (window_pool_attention_mma.cu).
//
// For the token at position p of a request (W = window, P = pool):
//   q  = rot_p(rmsnorm_all(q_proj) * gq),  k_p = rot_p(rmsnorm_all(k_proj) * gk)   over ALL heads' columns
//   v_p = turn_p(v_proj)                                                           over all of a value head
//   tokens seen:  j with 0 <= p - j < W           (all j <= p when W = 0)
//   blocks seen:  b with b*P + P - 1 <= p - W, key = mean_j k_j, value = mean_j v_j over its P tokens,
//                 as the cache holds them
//   out = turn_{-p}( softmax(scale * q.[keys]) [values] ),   one softmax over blocks and tokens
// rot turns the pairs (i, i + R/2) of the first R dimensions of a head by p * f_i, cos and sin
// times an amplitude; turn does the same over all of a value head with its own frequencies.
//
// Cache layout (parts/base.py, KeyValuePlanesSpec): a page holds `rows` rows, keys first
// ([kv_heads, rows, key_dim]) then values ([kv_heads, rows, value_dim]).  The token cache has a
// row per token; the block cache a row per P tokens, row b of a request on page
// table[b / rows] at offset b % rows.
#include "common.cuh"
#include "planes.cuh"

namespace si {

// ---------------------------------------------------------------- prepare
// One block per token.  qkv row: [H*kd queries | G*kd keys | G*vd values].  Queries are
// normalised and rotated in place; keys and values go to the token cache at `slots[t]`
// (page * rows + offset).
template <typename T, typename TW>
__global__ void wp_prepare_kernel(T* __restrict__ qkv, int stride, const int* __restrict__ positions,
                                  const TW* __restrict__ q_gain, const TW* __restrict__ k_gain,
                                  const float* __restrict__ freq_qk, float amp, int rot_dims,
                                  const float* __restrict__ freq_v, const int* __restrict__ slots,
                                  T* __restrict__ pool, PlanesLayout lay, int H, float eps,
                                  int write_kv) {
  extern __shared__ float sm[];
  __shared__ float red[32];
  const int G = lay.kv_heads, kd = lay.kd, vd = lay.vd;
  const int nq = H * kd, nk = G * kd, nv = G * vd;
  float* row_s = sm;                       // [nq + nk + nv]
  float* cs_qk = row_s + nq + nk + nv;     // [rot_dims/2][2]
  float* cs_v = cs_qk + rot_dims;          // [vd/2][2] (freq_v may be null: no turning)
  const int t = blockIdx.x, tid = threadIdx.x;
  const int half = rot_dims / 2, vhalf = vd / 2;
  pdl_wait();
  pdl_trigger();
  const float pos = (float)positions[t];
  for (int i = tid; i < half; i += blockDim.x) {
    float s, c;
    sincosf(pos * freq_qk[i], &s, &c);
    cs_qk[2 * i] = c * amp;
    cs_qk[2 * i + 1] = s * amp;
  }
  if (freq_v)
    for (int i = tid; i < vhalf; i += blockDim.x) {
      float s, c;
      sincosf(pos * freq_v[i], &s, &c);
      cs_v[2 * i] = c;
      cs_v[2 * i + 1] = s;
    }
  T* row = qkv + (size_t)t * stride;
  float sq = 0.0f, sk = 0.0f;
  for (int i = tid; i < nq + nk + nv; i += blockDim.x) {
    const float x = to_f32<T>(row[i]);
    row_s[i] = x;
    if (i < nq) sq += x * x;
    else if (i < nq + nk) sk += x * x;
  }
  const float tq = block_sum(sq, red);
  const float tk = block_sum(sk, red);
  const float rq = rsqrtf(tq / (float)nq + eps), rk = rsqrtf(tk / (float)nk + eps);
  const int slot = write_kv ? slots[t] : 0;
  const int page = slot / lay.rows, off = slot - page * lay.rows;
  // queries and keys: normalise, then turn the first rot_dims dimensions of each head
  for (int e = tid; e < nq + nk; e += blockDim.x) {
    const bool is_q = e < nq;
    const int idx = is_q ? e : e - nq;
    const int head = idx / kd, i = idx - head * kd;
    const float r = is_q ? rq : rk;
    const TW* gain = is_q ? q_gain : k_gain;
    float x = (row_s[e] * r) * to_f32<TW>(gain[idx]);
    if (i < rot_dims) {
      const int pi = i < half ? i + half : i - half;
      const float y = (row_s[e - i + pi] * r) * to_f32<TW>(gain[idx - i + pi]);
      const int fi = i < half ? i : i - half;
      const float c = cs_qk[2 * fi], s = cs_qk[2 * fi + 1];
      x = i < half ? x * c - y * s : x * c + y * s;
    }
    if (is_q) row[e] = from_f32<T>(x);
    else if (write_kv) pool[lay.key_at(page, head, off) + i] = from_f32<T>(x);
  }
  if (write_kv) {
    for (int e = tid; e < nv; e += blockDim.x) {
      const int head = e / vd, i = e - head * vd;
      float x = row_s[nq + nk + e];
      if (freq_v && i < 2 * vhalf) {
        const int pi = i < vhalf ? i + vhalf : i - vhalf;
        const float y = row_s[nq + nk + e - i + pi];
        const int fi = i < vhalf ? i : i - vhalf;
        const float c = cs_v[2 * fi], s = cs_v[2 * fi + 1];
        x = i < vhalf ? x * c - y * s : x * c + y * s;
      }
      pool[lay.value_at(page, head, off) + i] = from_f32<T>(x);
    }
  }
}

// ------------------------------------------------------------------- pool
// One block per (token, kv head).  The token that ends block b (position b*P + P - 1) makes
// the block's row: the mean of its P keys and of its P values, read back from the token cache.
template <typename T>
__global__ void wp_pool_kernel(const int* __restrict__ positions, const int* __restrict__ tok_seq,
                               const T* __restrict__ tok_pool, const int* __restrict__ tok_table,
                               int tok_table_stride, PlanesLayout tl, T* __restrict__ blk_pool,
                               const int* __restrict__ blk_table, int blk_table_stride,
                               PlanesLayout bl, int P) {
  const int t = blockIdx.x, g = blockIdx.y;
  pdl_wait();
  pdl_trigger();
  const int p = positions[t];
  if ((p + 1) % P != 0) return;
  const int b = p / P, seq = tok_seq[t];
  const int* tt = tok_table + (size_t)seq * tok_table_stride;
  const int bpage = blk_table[(size_t)seq * blk_table_stride + b / bl.rows];
  const int brow = b % bl.rows;
  for (int i = threadIdx.x; i < tl.kd + tl.vd; i += blockDim.x) {
    float sum = 0.0f;
    for (int j = b * P; j <= p; ++j) {
      const int page = tt[j / tl.rows], off = j % tl.rows;
      sum += i < tl.kd ? to_f32<T>(tok_pool[tl.key_at(page, g, off) + i])
                       : to_f32<T>(tok_pool[tl.value_at(page, g, off) + i - tl.kd]);
    }
    if (i < tl.kd) blk_pool[bl.key_at(bpage, g, brow) + i] = from_f32<T>(sum / (float)P);
    else blk_pool[bl.value_at(bpage, g, brow) + i - tl.kd] = from_f32<T>(sum / (float)P);
  }
}

// -------------------------------------------------------------- attention
constexpr int WP_THREADS = 128;

template <typename T>
__device__ __forceinline__ float dot_any(const float* __restrict__ qs, const T* __restrict__ krow,
                                         int n) {
  float acc = 0.0f;
  for (int d = 0; d < n; ++d) acc = fmaf(qs[d], to_f32<T>(krow[d]), acc);
  return acc;
}

// One block per (token, query head).  The keys are numbered x = 0..nb-1 (blocks) and then
// nb.. (tokens lo..p); they are visited in tiles of WP_THREADS of that numbering, which
// depends on the position alone, so a token's result does not depend on the batch or the cut.
template <typename T>
__global__ void __launch_bounds__(WP_THREADS)
wp_attention_kernel(const T* __restrict__ q, int q_stride, const int* __restrict__ positions,
                    const int* __restrict__ tok_seq, const T* __restrict__ tok_pool,
                    const int* __restrict__ tok_table, int tok_table_stride, PlanesLayout tl,
                    const T* __restrict__ blk_pool, const int* __restrict__ blk_table,
                    int blk_table_stride, PlanesLayout bl, T* __restrict__ out, int out_stride,
                    int H, float scale, int W, int P, const float* __restrict__ freq_v) {
  extern __shared__ float sm[];
  const int kd = tl.kd, vd = tl.vd;
  float* qs = sm;                  // [kd]
  float* ps = qs + kd;             // [WP_THREADS]
  float* os = ps + WP_THREADS;     // [vd]
  long long* voff = reinterpret_cast<long long*>(sm + ((kd + WP_THREADS + vd + 1) & ~1));  // [WP_THREADS]
  __shared__ float red[32];
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  pdl_wait();
  const int pos = positions[t], seq = tok_seq[t];
  const int g = h / (H / tl.kv_heads);
  const int lo = (W > 0 && pos - W + 1 > 0) ? pos - W + 1 : 0;
  const int nb = (W > 0 && P > 0 && pos - W + 1 > 0) ? (pos - W + 1) / P : 0;
  const int n_keys = nb + pos - lo + 1;
  const T* qrow = q + (size_t)t * q_stride + (size_t)h * kd;
  for (int d = tid; d < kd; d += WP_THREADS) qs[d] = to_f32<T>(qrow[d]);
  __syncthreads();
  const int* ttab = tok_table + (size_t)seq * tok_table_stride;
  const int* btab = blk_table ? blk_table + (size_t)seq * blk_table_stride : nullptr;

  float m_run = -INFINITY, l_run = 0.0f, acc0 = 0.0f, acc1 = 0.0f;
  for (int x0 = 0; x0 < n_keys; x0 += WP_THREADS) {
    const int x = x0 + tid;
    const int n_here = min(WP_THREADS, n_keys - x0);
    float s = -INFINITY;
    if (x < n_keys) {
      const T* krow;
      if (x < nb) {
        const int page = btab[x / bl.rows], row = x % bl.rows;
        krow = blk_pool + bl.key_at(page, g, row);
        voff[tid] = -(bl.value_at(page, g, row) + 1);  // negative: in the block cache
      } else {
        const int j = lo + (x - nb);
        const int page = ttab[j / tl.rows], row = j % tl.rows;
        krow = tok_pool + tl.key_at(page, g, row);
        voff[tid] = tl.value_at(page, g, row);
      }
      s = dot_any<T>(qs, krow, kd) * scale;
    }
    const float m_new = fmaxf(m_run, block_max(s, red));
    const float p = (x < n_keys) ? expf(s - m_new) : 0.0f;
    ps[tid] = p;
    const float p_sum = block_sum(p, red);  // its barriers also publish ps and voff
    const float alpha = (m_run == -INFINITY) ? 0.0f : expf(m_run - m_new);
    l_run = l_run * alpha + p_sum;
    m_run = m_new;
    acc0 *= alpha;
    acc1 *= alpha;
    for (int jj = 0; jj < n_here; ++jj) {
      const long long vo = voff[jj];
      const T* vrow = vo < 0 ? blk_pool + (-vo - 1) : tok_pool + vo;
      const float pj = ps[jj];
      if (tid < vd) acc0 = fmaf(pj, to_f32<T>(vrow[tid]), acc0);
      if (tid + WP_THREADS < vd) acc1 = fmaf(pj, to_f32<T>(vrow[tid + WP_THREADS]), acc1);
    }
    __syncthreads();  // ps and voff are rewritten by the next tile
  }
  pdl_trigger();
  const float inv_l = 1.0f / l_run;
  if (tid < vd) os[tid] = acc0 * inv_l;
  if (tid + WP_THREADS < vd) os[tid + WP_THREADS] = acc1 * inv_l;
  __syncthreads();
  // turn the head's output back by -pos
  T* orow = out + (size_t)t * out_stride + (size_t)h * vd;
  const int vhalf = vd / 2;
  for (int i = tid; i < vd; i += WP_THREADS) {
    float x = os[i];
    if (freq_v && i < 2 * vhalf) {
      const int fi = i < vhalf ? i : i - vhalf;
      float s, c;
      sincosf((float)pos * freq_v[fi], &s, &c);
      const float y = os[i < vhalf ? i + vhalf : i - vhalf];
      x = i < vhalf ? x * c + y * s : x * c - y * s;
    }
    orow[i] = from_f32<T>(x);
  }
}

}  // namespace si

static int wp_layout_ok(int kv_heads, int rows, int kd, int vd) {
  return kv_heads > 0 && rows > 0 && kd > 0 && vd > 0;
}

// gains: gain_dtype (0 float32, 1 bfloat16).  freq_v null: values are stored as projected.
SI_API int si_wp_prepare(void* qkv, int stride, const int* positions, const void* q_gain,
                         const void* k_gain, int gain_dtype, const float* freq_qk, float amp,
                         int rot_dims, const float* freq_v, const int* slots, void* pool,
                         int n_tokens, int H, int G, int kd, int vd, int rows, float eps,
                         int write_kv, int dtype, cudaStream_t stream) {
  if (!qkv || !positions || !q_gain || !k_gain || n_tokens < 0 || H <= 0 || !(eps > 0.0f))
    return SI_ERR_ARG;
  if (!wp_layout_ok(G, rows, kd, vd) || rot_dims < 0 || rot_dims > kd || rot_dims % 2 != 0)
    return SI_ERR_ARG;
  if ((rot_dims > 0 && !freq_qk) || (write_kv && (!slots || !pool))) return SI_ERR_ARG;
  if (n_tokens == 0) return SI_OK;
  si::PlanesLayout lay{G, rows, kd, vd};
  const int width = (H + G) * kd + G * vd;
  const size_t smem = (size_t)(width + rot_dims + vd + 2) * sizeof(float);
  if (smem > 200 * 1024) return SI_ERR_TOO_LARGE;
  int threads = (width / 4 + 31) / 32 * 32;
  threads = threads > 512 ? 512 : (threads < 64 ? 64 : threads);
#define SI_WP_PREP(T, TW)                                                                          \
  do {                                                                                             \
    auto kern = si::wp_prepare_kernel<T, TW>;                                                      \
    if (smem > 48 * 1024) SI_ALLOW_DYNAMIC_SMEM(kern, smem);                                       \
    SI_LAUNCH(kern, n_tokens, threads, smem, stream, (T*)qkv, stride, positions, (const TW*)q_gain, \
              (const TW*)k_gain, freq_qk, amp, rot_dims, freq_v, slots, (T*)pool, lay, H, eps,     \
              write_kv);                                                                           \
  } while (0)
  if (dtype == SI_BF16 && gain_dtype == SI_BF16) SI_WP_PREP(__nv_bfloat16, __nv_bfloat16);
  else if (dtype == SI_BF16 && gain_dtype == SI_F32) SI_WP_PREP(__nv_bfloat16, float);
  else if (dtype == SI_F32 && gain_dtype == SI_F32) SI_WP_PREP(float, float);
  else return SI_ERR_DTYPE;
#undef SI_WP_PREP
  return SI_OK;
}

SI_API int si_wp_pool(const int* positions, const int* tok_seq, const void* tok_pool,
                      const int* tok_table, int tok_table_stride, int tok_rows, void* blk_pool,
                      const int* blk_table, int blk_table_stride, int blk_rows, int n_tokens, int G,
                      int kd, int vd, int P, int dtype, cudaStream_t stream) {
  if (!positions || !tok_seq || !tok_pool || !tok_table || !blk_pool || !blk_table || n_tokens < 0 ||
      P <= 0 || !wp_layout_ok(G, tok_rows, kd, vd) || blk_rows <= 0)
    return SI_ERR_ARG;
  if (G > 65535) return SI_ERR_TOO_LARGE;
  if (n_tokens == 0) return SI_OK;
  si::PlanesLayout tl{G, tok_rows, kd, vd}, bl{G, blk_rows, kd, vd};
  dim3 grid(n_tokens, G);
  int threads = (kd + vd + 31) / 32 * 32;
  threads = threads > 256 ? 256 : threads;
  if (dtype == SI_BF16)
    SI_LAUNCH(si::wp_pool_kernel<__nv_bfloat16>, grid, threads, 0, stream, positions, tok_seq,
              (const __nv_bfloat16*)tok_pool, tok_table, tok_table_stride, tl,
              (__nv_bfloat16*)blk_pool, blk_table, blk_table_stride, bl, P);
  else if (dtype == SI_F32)
    SI_LAUNCH(si::wp_pool_kernel<float>, grid, threads, 0, stream, positions, tok_seq,
              (const float*)tok_pool, tok_table, tok_table_stride, tl, (float*)blk_pool, blk_table,
              blk_table_stride, bl, P);
  else
    return SI_ERR_DTYPE;
  return SI_OK;
}

// W <= 0: every earlier token is seen (and no block); P <= 0 or blk_pool null: no blocks.
SI_API int si_wp_attention(const void* q, int q_stride, const int* positions, const int* tok_seq,
                           const void* tok_pool, const int* tok_table, int tok_table_stride,
                           int tok_rows, const void* blk_pool, const int* blk_table,
                           int blk_table_stride, int blk_rows, void* out, int out_stride,
                           int n_tokens, int H, int G, int kd, int vd, float scale, int W, int P,
                           const float* freq_v, int dtype, cudaStream_t stream) {
  if (!q || !positions || !tok_seq || !tok_pool || !tok_table || !out || n_tokens < 0 || H <= 0)
    return SI_ERR_ARG;
  if (!wp_layout_ok(G, tok_rows, kd, vd) || H % G != 0) return SI_ERR_ARG;
  if (P > 0 && W > 0 && (!blk_pool || !blk_table || blk_rows <= 0)) return SI_ERR_ARG;
  if (vd > 2 * si::WP_THREADS) return SI_ERR_UNSUPPORTED;
  if (H > 65535) return SI_ERR_TOO_LARGE;
  if (n_tokens == 0) return SI_OK;
  if (!blk_pool) P = 0;
  si::PlanesLayout tl{G, tok_rows, kd, vd}, bl{G, blk_rows > 0 ? blk_rows : 1, kd, vd};
  dim3 grid(n_tokens, H);
  const size_t smem = (size_t)(kd + si::WP_THREADS + vd + 2) * sizeof(float) +
                      si::WP_THREADS * sizeof(long long);
  if (smem > 48 * 1024) return SI_ERR_TOO_LARGE;
  if (dtype == SI_BF16)
    SI_LAUNCH(si::wp_attention_kernel<__nv_bfloat16>, grid, si::WP_THREADS, smem, stream,
              (const __nv_bfloat16*)q, q_stride, positions, tok_seq, (const __nv_bfloat16*)tok_pool,
              tok_table, tok_table_stride, tl, (const __nv_bfloat16*)blk_pool, blk_table,
              blk_table_stride, bl, (__nv_bfloat16*)out, out_stride, H, scale, W, P, freq_v);
  else if (dtype == SI_F32)
    SI_LAUNCH(si::wp_attention_kernel<float>, grid, si::WP_THREADS, smem, stream, (const float*)q,
              q_stride, positions, tok_seq, (const float*)tok_pool, tok_table, tok_table_stride, tl,
              (const float*)blk_pool, blk_table, blk_table_stride, bl, (float*)out, out_stride, H,
              scale, W, P, freq_v);
  else
    return SI_ERR_DTYPE;
  return SI_OK;
}
