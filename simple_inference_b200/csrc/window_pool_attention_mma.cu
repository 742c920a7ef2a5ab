// Window attention with pooled blocks on the tensor cores (bfloat16 storage, mma.sync
// m16n8k16 with float32 accumulation; scores, softmax and the output sums are float32, and the
// softmax weights enter the second product as two bfloat16 terms).
//
// A block works one tile of 16 consecutive tokens of one sequence for one key/value head; each
// of its warps is one query head of that group, so the group's heads share every key and value
// the block fetches.  The keys a tile can see are numbered x = 0 .. nb-1 (pooled blocks, nb
// those seen by the tile's last token) and then the tokens from the first one that the tile's
// first token sees to the tile's last token; they stream through a ring of shared-memory stages of 64
// keys (cp.async through the page tables of both caches), and each row masks what it does not
// see: blocks not yet wholly before ITS window, tokens before its window or after itself.
// Where a tile's tokens times the group's heads fill no more than the 16 rows of one fragment
// (a sequence that brings one token: decoding), the rows are (token, head) pairs, every warp
// holds all of them and takes every n-th run of 16 keys of a stage; the warps' partial results
// (row maximum, sum and output) are joined through shared memory at the end.  Such tiles can also
// be shared out among several blocks (every n-th stage each) that leave their partial results in
// scratch memory for a small second kernel to join: a decode step has too few (request, key/value
// head) pairs to fill the GPU otherwise.
// The same formulas as the generic kernel (window_pool_attention.cu), which stays the kernel of
// float32 models and of head sizes that are no multiple of 16 or above 128.
#include "common.cuh"
#include "planes.cuh"

namespace si {

typedef __nv_bfloat16 bf16;

constexpr int WPM_QT = 16;      // query rows of a tile
constexpr int WPM_KT = 64;      // keys per stage
constexpr int WPM_NST = 3;      // stages: a tile with few rows spends less on a stage than its copy takes
constexpr int WPM_PAD = 8;      // elements added to a shared-memory row: no bank conflicts
constexpr int WPM_MAX_WARPS = 4;
constexpr int WPM_PAGES = 1024;  // page numbers of a tile kept in shared memory

__device__ __forceinline__ void wpm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void wpm_ldmatrix_x4_trans(uint32_t (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void wpm_ldmatrix_x4(uint32_t (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void wpm_cp16(void* dst, const void* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ uint32_t wpm_pack(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// KD16: 16-wide steps of a key head the kernel has registers for; VD8: 8-wide tiles of a value
// head.  The real sizes (multiples of 16, no larger) come in the layouts.
template <int KD16, int VD8>
__global__ void __launch_bounds__(32 * WPM_MAX_WARPS)
wp_attention_mma_kernel(const bf16* __restrict__ q, int q_stride, const int* __restrict__ positions,
                        const int* __restrict__ cu_q, int n_seqs, const bf16* __restrict__ tok_pool,
                        const int* __restrict__ tok_table, int tok_table_stride, PlanesLayout tl,
                        const bf16* __restrict__ blk_pool, const int* __restrict__ blk_table,
                        int blk_table_stride, PlanesLayout bl, bf16* __restrict__ out, int out_stride,
                        int H, float scale, int W, int P, const float* __restrict__ freq_v,
                        int key_splits, float* __restrict__ scratch) {
  extern __shared__ __align__(16) unsigned char wpm_smem[];
  const int kd = tl.kd, vd = tl.vd, G = tl.kv_heads;
  const int kstride = kd + WPM_PAD, vstride = vd + WPM_PAD;
  bf16* k_s = reinterpret_cast<bf16*>(wpm_smem);          // [NST][KT][kstride]
  bf16* v_s = k_s + WPM_NST * WPM_KT * kstride;           // [NST][KT][vstride]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, tq = lane & 3;                // row and column pair within a fragment

  // which tile: sequences in order, ceil(tokens / 16) tiles each (the step's description was
  // on the device before the step's first kernel)
  int seq = -1, t0 = 0, nq = 0;
  {
    int b = blockIdx.x;
    for (int s = 0; s < n_seqs; ++s) {
      const int a = cu_q[s], e = cu_q[s + 1];
      const int nt = (e - a + WPM_QT - 1) / WPM_QT;
      if (b < nt) {
        seq = s;
        t0 = a + b * WPM_QT;
        nq = min(WPM_QT, e - t0);
        break;
      }
      b -= nt;
    }
  }
  if (seq < 0) return;
  const int g = blockIdx.y, Hg = H / G;
  const int nw = (int)(blockDim.x >> 5);
  // few rows: all heads of the group in one fragment, the warps share out the keys
  const bool split = nw > 1 && nq * Hg <= WPM_QT;
  const int Z = split ? key_splits : 1, zi = split ? (int)blockIdx.z : 0;   // blocks that share the stages
  if (split ? (int)blockIdx.z >= Z : (int)blockIdx.z * nw >= Hg) return;
  const int head_in_group = blockIdx.z * nw + warp;
  const bool active = split || head_in_group < Hg;
  const int n_rows = split ? nq * Hg : nq;
  auto row_tok = [&](int r) { return split ? r / Hg : r; };          // token of a fragment row
  auto row_head = [&](int r) { return g * Hg + (split ? r % Hg : head_in_group); };
  const int p0 = positions[t0], p_last = p0 + nq - 1;
  const int lo_min = (W > 0 && p0 - W + 1 > 0) ? p0 - W + 1 : 0;
  const int nb_max = (W > 0 && P > 0 && p_last - W + 1 > 0) ? (p_last - W + 1) / P : 0;
  const int n_slots = nb_max + (p_last - lo_min + 1);
  const int all_tiles = (n_slots + WPM_KT - 1) / WPM_KT;
  const int n_tiles = zi < all_tiles ? (all_tiles - zi + Z - 1) / Z : 0;   // this block's: zi, zi+Z, ...
  const int* ttab = tok_table + (size_t)seq * tok_table_stride;
  const int* btab = blk_table ? blk_table + (size_t)seq * blk_table_stride : nullptr;
  // the page numbers the tile will ask for, side by side in shared memory (a look-up in the
  // tables themselves would put a trip to memory before every copy): token pages from the
  // first one seen, then block pages
  __shared__ int pages_s[WPM_PAGES];
  const int tp0 = lo_min / tl.rows, n_tp = p_last / tl.rows - tp0 + 1;
  const int n_bp = nb_max > 0 ? (nb_max - 1) / bl.rows + 1 : 0;
  const bool staged = n_tp + n_bp <= WPM_PAGES;
  if (staged) {
    for (int i = tid; i < n_tp; i += blockDim.x) pages_s[i] = ttab[tp0 + i];
    for (int i = tid; i < n_bp; i += blockDim.x) pages_s[n_tp + i] = btab[i];
  }
  __syncthreads();
  pdl_wait();

  // Eight threads copy one row of a stage (a key and its value, 16 bytes at a time), so a
  // row's page is looked up once by each of them.
  const int row_lane = tid >> 3, ch_lane = tid & 7, rows_per_pass = (int)blockDim.x >> 3;
  auto load_tile = [&](int own_i) {   // the block's own_i-th stage of keys
    const int st = own_i % WPM_NST;
    const int i = zi + own_i * Z;
    const int kchunks = kd >> 3, per_row = (kd + vd) >> 3;
    for (int row = row_lane; row < WPM_KT; row += rows_per_pass) {
      const int x = i * WPM_KT + row;
      bf16* kdst = k_s + (st * WPM_KT + row) * kstride;
      bf16* vdst = v_s + (st * WPM_KT + row) * vstride;
      if (x < n_slots) {
        const bf16 *ksrc, *vsrc;
        if (x < nb_max) {
          const int lp = x / bl.rows, r = x - lp * bl.rows;
          const int page = staged ? pages_s[n_tp + lp] : btab[lp];
          ksrc = blk_pool + bl.key_at(page, g, r);
          vsrc = blk_pool + bl.value_at(page, g, r);
        } else {
          const int j = lo_min + (x - nb_max);
          const int lp = j / tl.rows, r = j - lp * tl.rows;
          const int page = staged ? pages_s[lp - tp0] : ttab[lp];
          ksrc = tok_pool + tl.key_at(page, g, r);
          vsrc = tok_pool + tl.value_at(page, g, r);
        }
        for (int c = ch_lane; c < per_row; c += 8) {
          if (c < kchunks) wpm_cp16(kdst + c * 8, ksrc + c * 8);
          else wpm_cp16(vdst + (c - kchunks) * 8, vsrc + (c - kchunks) * 8);
        }
      } else {
        for (int c = ch_lane; c < per_row; c += 8) {   // a value row must not be garbage
          if (c < kchunks) *reinterpret_cast<uint4*>(kdst + c * 8) = make_uint4(0, 0, 0, 0);
          else *reinterpret_cast<uint4*>(vdst + (c - kchunks) * 8) = make_uint4(0, 0, 0, 0);
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

#pragma unroll
  for (int i = 0; i < WPM_NST - 1; ++i) {
    if (i < n_tiles) load_tile(i);
    else asm volatile("cp.async.commit_group;" ::: "memory");
  }

  // this warp's queries as A fragments: rows gq and gq+8 of the tile, all of the head's columns
  uint32_t qf[KD16][4];
#pragma unroll
  for (int kk = 0; kk < KD16; ++kk) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int row = gq + (e & 1) * 8, col = kk * 16 + tq * 2 + (e >> 1) * 8;
      uint32_t v = 0;
      if (active && row < n_rows && col < kd)
        v = *reinterpret_cast<const uint32_t*>(q + (size_t)(t0 + row_tok(row)) * q_stride +
                                               (size_t)row_head(row) * kd + col);
      qf[kk][e] = v;
    }
  }
  // what each of this thread's two rows sees
  int p_row[2], nb_row[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    p_row[r] = p0 + row_tok(gq + r * 8);
    nb_row[r] = (W > 0 && P > 0 && p_row[r] - W + 1 > 0) ? (p_row[r] - W + 1) / P : 0;
  }
  // which runs of 16 keys of a stage are this warp's (all of them unless the warps share them out)
  unsigned own = 0;
#pragma unroll
  for (int kk = 0; kk < WPM_KT / 16; ++kk)
    if (!split || kk % nw == warp) own |= 1u << kk;
  // a stage needs no masking when every row sees all of it: its blocks are seen by the first
  // token already, its tokens lie inside the last token's window and not after the first token
  const int nb_first = (W > 0 && P > 0 && p0 - W + 1 > 0) ? (p0 - W + 1) / P : 0;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
  float o[VD8][4];
#pragma unroll
  for (int n = 0; n < VD8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[n][e] = 0.0f;

  for (int i = 0; i < n_tiles; ++i) {
    if (i + WPM_NST - 1 < n_tiles) load_tile(i + WPM_NST - 1);   // into the stage tile i-1 has left
    else asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group %0;" ::"n"(WPM_NST - 1) : "memory");
    __syncthreads();
    if (active) {
      const bf16* ks = k_s + (i % WPM_NST) * WPM_KT * kstride;
      const bf16* vs = v_s + (i % WPM_NST) * WPM_KT * vstride;
      float s[WPM_KT / 8][4];
      const unsigned k_base = (unsigned)__cvta_generic_to_shared(ks);
#pragma unroll
      for (int nt = 0; nt < WPM_KT / 8; nt += 2) {
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] = s[nt + 1][e] = 0.0f;
        if (!((own >> (nt >> 1)) & 1)) continue;   // another warp's run of 16 keys
#pragma unroll
        for (int kk = 0; kk < KD16; ++kk) {
          if (kk * 16 < kd) {
            // four 8x8 pieces: keys nt*8.. and (nt+1)*8.., each with the step's two halves
            const int key = (nt + (lane >> 4)) * 8 + (lane & 7);
            uint32_t b[4];
            wpm_ldmatrix_x4(b, k_base + (unsigned)((key * kstride + kk * 16 + ((lane >> 3) & 1) * 8) * 2));
            wpm_mma(s[nt], qf[kk], b[0], b[1]);
            wpm_mma(s[nt + 1], qf[kk], b[2], b[3]);
          }
        }
      }
      // scale and mask; row maxima
      float mx[2] = {-INFINITY, -INFINITY};
      const int x0 = (zi + i * Z) * WPM_KT, x1 = x0 + WPM_KT - 1;   // the stage's first and last slot
      bool all_seen = x1 < n_slots;   // (rows past the tile's last are never stored)
      if (x0 < nb_max) all_seen = all_seen && x1 < nb_first;
      else all_seen = all_seen && lo_min + (x1 - nb_max) <= p0 &&
                      (W <= 0 || lo_min + (x0 - nb_max) > p_last - W);
#pragma unroll
      for (int nt = 0; nt < WPM_KT / 8; ++nt) {
        if (!((own >> (nt >> 1)) & 1)) continue;   // not this warp's keys: neither masked nor summed
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = e >> 1;
          bool vis = true;
          if (!all_seen) {
            const int x = x0 + nt * 8 + tq * 2 + (e & 1);
            if (x < nb_max) {
              vis = vis && x < nb_row[r];
            } else {
              const int j = lo_min + (x - nb_max);
              vis = vis && j <= p_row[r] && (W <= 0 || j > p_row[r] - W);
            }
            vis = vis && x < n_slots && gq + r * 8 < n_rows;
          }
          const float v = vis ? s[nt][e] * scale : -INFINITY;
          s[nt][e] = v;
          mx[r] = fmaxf(mx[r], v);
        }
      }
      float alpha[2], m_use[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m_run[r], mx[r]);
        m_use[r] = m_new == -INFINITY ? 0.0f : m_new;     // a row that has seen nothing yet
        alpha[r] = __expf(m_run[r] - m_use[r]);            // exp(-inf) = 0 on the first tile
        m_run[r] = m_new;
        l_run[r] *= alpha[r];
      }
#pragma unroll
      for (int n = 0; n < VD8; ++n) {
        o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
        o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
      }
#pragma unroll
      for (int nt = 0; nt < WPM_KT / 8; ++nt) {
        if (!((own >> (nt >> 1)) & 1)) continue;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pv = __expf(s[nt][e] - m_use[e >> 1]);
          s[nt][e] = pv;
          l_run[e >> 1] += pv;
        }
      }
      // O += P V, 16 keys at a time; V fragments come transposed out of shared memory
#pragma unroll
      for (int kk = 0; kk < WPM_KT / 16; ++kk) {
        if (!((own >> kk) & 1)) continue;
        // the weights as two bfloat16 terms, p = hi + lo: what the tensor cores multiply keeps 16
        // bits of the float32 weight instead of 8
        uint32_t pa[4], pb[4];
#pragma unroll
        for (int f = 0; f < 4; ++f) {
          const float w0 = s[2 * kk + (f >> 1)][(f & 1) * 2], w1 = s[2 * kk + (f >> 1)][(f & 1) * 2 + 1];
          const __nv_bfloat162 hi = __floats2bfloat162_rn(w0, w1);
          const float2 back = __bfloat1622float2(hi);
          pa[f] = *reinterpret_cast<const uint32_t*>(&hi);
          pb[f] = wpm_pack(w0 - back.x, w1 - back.y);
        }
        const int key = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
        for (int n2 = 0; n2 < VD8 / 2; ++n2) {
          if (n2 * 16 < vd) {
            const bf16* vp = vs + key * vstride + n2 * 16 + (lane >> 4) * 8;
            uint32_t b[4];
            wpm_ldmatrix_x4_trans(b, (unsigned)__cvta_generic_to_shared(vp));
            wpm_mma(o[2 * n2], pa, b[0], b[1]);
            wpm_mma(o[2 * n2 + 1], pa, b[2], b[3]);
            wpm_mma(o[2 * n2], pb, b[0], b[1]);
            wpm_mma(o[2 * n2 + 1], pb, b[2], b[3]);
          }
        }
      }
    }
    __syncthreads();   // the stage may be refilled
  }
  pdl_trigger();
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  float* smem_f = reinterpret_cast<float*>(wpm_smem);
  const int vhalf = vd >> 1;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  if (!split) {
    // normalise, hand the warp's rows to shared memory, turn them back by their positions, store
    float* o_s = smem_f + warp * WPM_QT * vd;   // [16][vd] of this warp
    if (active) {
      const float inv0 = 1.0f / l_run[0], inv1 = 1.0f / l_run[1];
#pragma unroll
      for (int n = 0; n < VD8; ++n) {
        if (n * 8 < vd) {
          const int col = n * 8 + tq * 2;
          o_s[gq * vd + col] = o[n][0] * inv0;
          o_s[gq * vd + col + 1] = o[n][1] * inv0;
          o_s[(gq + 8) * vd + col] = o[n][2] * inv1;
          o_s[(gq + 8) * vd + col + 1] = o[n][3] * inv1;
        }
      }
      __syncwarp();
      const int h = row_head(0);
      for (int idx = lane; idx < nq * vd; idx += 32) {
        const int row = idx / vd, d = idx - row * vd;
        float x = o_s[idx];
        if (freq_v) {
          const int fi = d < vhalf ? d : d - vhalf;
          float sn, cs;
          sincosf((float)(p0 + row) * freq_v[fi], &sn, &cs);
          const float y = o_s[row * vd + (d < vhalf ? d + vhalf : d - vhalf)];
          x = d < vhalf ? x * cs + y * sn : x * cs - y * sn;
        }
        out[(size_t)(t0 + row) * out_stride + (size_t)h * vd + d] = __float2bfloat16_rn(x);
      }
    }
    return;
  }
  // the warps' partial results side by side, then one pass that joins them, one that turns
  float* o_w = smem_f + warp * WPM_QT * vd;              // [nw][16][vd] unnormalised sums
  float* ml_s = smem_f + nw * WPM_QT * vd;               // [nw][16][2] row maximum and sum
  float* fin = ml_s + nw * WPM_QT * 2;                   // [16][vd] joined rows
#pragma unroll
  for (int n = 0; n < VD8; ++n) {
    if (n * 8 < vd) {
      const int col = n * 8 + tq * 2;
      o_w[gq * vd + col] = o[n][0];
      o_w[gq * vd + col + 1] = o[n][1];
      o_w[(gq + 8) * vd + col] = o[n][2];
      o_w[(gq + 8) * vd + col + 1] = o[n][3];
    }
  }
  if (tq == 0) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      ml_s[(warp * WPM_QT + gq + r * 8) * 2] = m_run[r];
      ml_s[(warp * WPM_QT + gq + r * 8) * 2 + 1] = l_run[r];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < n_rows * vd; idx += blockDim.x) {
    const int row = idx / vd, d = idx - row * vd;
    float m_all = -INFINITY;
    for (int w = 0; w < nw; ++w) m_all = fmaxf(m_all, ml_s[(w * WPM_QT + row) * 2]);
    float l_all = 0.0f, acc = 0.0f;
    for (int w = 0; w < nw; ++w) {   // fixed order
      const float m_w = ml_s[(w * WPM_QT + row) * 2];
      const float f = m_w == -INFINITY ? 0.0f : __expf(m_w - m_all);
      l_all = fmaf(ml_s[(w * WPM_QT + row) * 2 + 1], f, l_all);
      acc = fmaf(smem_f[(w * WPM_QT + row) * vd + d], f, acc);
    }
    if (Z > 1) {   // unnormalised, with its maximum and sum, for the joining kernel
      float* part = scratch + ((((size_t)blockIdx.x * G + g) * Z + zi) * WPM_QT + row) * (vd + 2);
      part[d] = acc;
      if (d == 0) {
        part[vd] = m_all;
        part[vd + 1] = l_all;
      }
    } else {
      fin[idx] = acc / l_all;
    }
  }
  if (Z > 1) return;
  __syncthreads();
  for (int idx = tid; idx < n_rows * vd; idx += blockDim.x) {
    const int row = idx / vd, d = idx - row * vd;
    const int tok = row_tok(row);
    float x = fin[idx];
    if (freq_v) {
      const int fi = d < vhalf ? d : d - vhalf;
      float sn, cs;
      sincosf((float)(p0 + tok) * freq_v[fi], &sn, &cs);
      const float y = fin[row * vd + (d < vhalf ? d + vhalf : d - vhalf)];
      x = d < vhalf ? x * cs + y * sn : x * cs - y * sn;
    }
    out[(size_t)(t0 + tok) * out_stride + (size_t)row_head(row) * vd + d] = __float2bfloat16_rn(x);
  }
}

// Joins what the blocks that shared a few-row tile's stages left in scratch memory, turns the
// rows back by their positions and stores them.  One block per (tile, key/value head).
__global__ void wp_attention_join_kernel(const float* __restrict__ scratch, const int* __restrict__ positions,
                                         const int* __restrict__ cu_q, int n_seqs, bf16* __restrict__ out,
                                         int out_stride, int H, int G, int vd, int warps, int key_splits,
                                         const float* __restrict__ freq_v) {
  extern __shared__ float join_s[];   // [rows][vd]
  int seq = -1, t0 = 0, nq = 0;
  {
    int b = blockIdx.x;
    for (int s = 0; s < n_seqs; ++s) {
      const int a = cu_q[s], e = cu_q[s + 1];
      const int nt = (e - a + WPM_QT - 1) / WPM_QT;
      if (b < nt) {
        seq = s;
        t0 = a + b * WPM_QT;
        nq = min(WPM_QT, e - t0);
        break;
      }
      b -= nt;
    }
  }
  const int g = blockIdx.y, Hg = H / G;
  if (seq < 0 || !(warps > 1 && nq * Hg <= WPM_QT)) return;   // not a tile that was shared out
  const int n_rows = nq * Hg, vhalf = vd >> 1, Z = key_splits;
  const int p0 = positions[t0];
  pdl_wait();
  pdl_trigger();
  const float* base = scratch + (((size_t)blockIdx.x * G + g) * Z) * WPM_QT * (vd + 2);
  for (int idx = threadIdx.x; idx < n_rows * vd; idx += blockDim.x) {
    const int row = idx / vd, d = idx - row * vd;
    float m_all = -INFINITY;
    for (int z = 0; z < Z; ++z) m_all = fmaxf(m_all, base[((size_t)z * WPM_QT + row) * (vd + 2) + vd]);
    float l_all = 0.0f, acc = 0.0f;
    for (int z = 0; z < Z; ++z) {   // fixed order
      const float* part = base + ((size_t)z * WPM_QT + row) * (vd + 2);
      const float f = part[vd] == -INFINITY ? 0.0f : __expf(part[vd] - m_all);
      l_all = fmaf(part[vd + 1], f, l_all);
      acc = fmaf(part[d], f, acc);
    }
    join_s[idx] = acc / l_all;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < n_rows * vd; idx += blockDim.x) {
    const int row = idx / vd, d = idx - row * vd;
    const int tok = row / Hg, h = g * Hg + row % Hg;
    float x = join_s[idx];
    if (freq_v) {
      const int fi = d < vhalf ? d : d - vhalf;
      float sn, cs;
      sincosf((float)(p0 + tok) * freq_v[fi], &sn, &cs);
      const float y = join_s[row * vd + (d < vhalf ? d + vhalf : d - vhalf)];
      x = d < vhalf ? x * cs + y * sn : x * cs - y * sn;
    }
    out[(size_t)(t0 + tok) * out_stride + (size_t)h * vd + d] = __float2bfloat16_rn(x);
  }
}

}  // namespace si

template <int KD16, int VD8>
static int launch_wp_attention_mma(const void* q, int q_stride, const int* positions, const int* cu_q,
                                   int n_seqs, const void* tok_pool, const int* tok_table,
                                   int tok_table_stride, si::PlanesLayout tl, const void* blk_pool,
                                   const int* blk_table, int blk_table_stride, si::PlanesLayout bl,
                                   void* out, int out_stride, int n_tokens, int H, float scale, int W,
                                   int P, const float* freq_v, int key_splits, float* scratch,
                                   cudaStream_t stream) {
  const int Hg = H / tl.kv_heads;
  const int warps = Hg < si::WPM_MAX_WARPS ? Hg : si::WPM_MAX_WARPS;
  const size_t stages = (size_t)si::WPM_NST * si::WPM_KT * (tl.kd + tl.vd + 2 * si::WPM_PAD) * sizeof(si::bf16);
  // joining the warps' partial results reuses the stages' memory and may need a little more
  const size_t join = (size_t)((warps + 1) * si::WPM_QT * tl.vd + warps * si::WPM_QT * 2) * sizeof(float);
  const size_t smem = stages > join ? stages : join;
  auto kern = si::wp_attention_mma_kernel<KD16, VD8>;
  if (smem > 48 * 1024) SI_ALLOW_DYNAMIC_SMEM(kern, smem);
  // an upper bound of the tiles: every sequence's last tile may be short
  const int chunks = (Hg + warps - 1) / warps;
  dim3 grid((n_tokens + si::WPM_QT - 1) / si::WPM_QT + n_seqs, tl.kv_heads,
            chunks > key_splits ? chunks : key_splits);
  SI_LAUNCH(kern, grid, 32 * warps, smem, stream, (const si::bf16*)q, q_stride, positions, cu_q, n_seqs,
            (const si::bf16*)tok_pool, tok_table, tok_table_stride, tl, (const si::bf16*)blk_pool,
            blk_table, blk_table_stride, bl, (si::bf16*)out, out_stride, H, scale, W, P, freq_v,
            key_splits, scratch);
  if (key_splits > 1) {
    dim3 jgrid(grid.x, tl.kv_heads);
    SI_LAUNCH(si::wp_attention_join_kernel, jgrid, 128, (size_t)si::WPM_QT * tl.vd * sizeof(float), stream,
              (const float*)scratch, positions, cu_q, n_seqs, (si::bf16*)out, out_stride, H, tl.kv_heads,
              tl.vd, warps, key_splits, freq_v);
  }
  return SI_OK;
}

// Whether the tensor-core kernel takes these head sizes (bfloat16 only).
SI_API int si_wp_attention_mma_fits(int kd, int vd) {
  return kd > 0 && vd > 0 && kd % 16 == 0 && vd % 16 == 0 && kd <= 128 && vd <= 128;
}

// Arguments as si_wp_attention, plus the sequences' token ranges cu_q[0..n_seqs]; bfloat16.
// key_splits > 1: tiles of few rows (tokens x heads of a group <= 16) are shared out among that
// many blocks and joined by a second kernel; scratch then holds
// (ceil(n_tokens / 16) + n_seqs) * G * key_splits * 16 * (vd + 2) floats.
SI_API int si_wp_attention_mma(const void* q, int q_stride, const int* positions, const int* cu_q,
                               int n_seqs, const void* tok_pool, const int* tok_table,
                               int tok_table_stride, int tok_rows, const void* blk_pool,
                               const int* blk_table, int blk_table_stride, int blk_rows, void* out,
                               int out_stride, int n_tokens, int H, int G, int kd, int vd, float scale,
                               int W, int P, const float* freq_v, int key_splits, float* scratch,
                               cudaStream_t stream) {
  if (key_splits < 1 || key_splits > 16 || (key_splits > 1 && !scratch)) return SI_ERR_ARG;
  if (!q || !positions || !cu_q || !tok_pool || !tok_table || !out || n_tokens < 0 || n_seqs < 0 ||
      H <= 0 || G <= 0 || H % G != 0 || tok_rows <= 0)
    return SI_ERR_ARG;
  if (!si_wp_attention_mma_fits(kd, vd)) return SI_ERR_UNSUPPORTED;
  if (P > 0 && W > 0 && (!blk_pool || !blk_table || blk_rows <= 0)) return SI_ERR_ARG;
  if (q_stride % 2 != 0 || ((uintptr_t)q & 3) || ((uintptr_t)tok_pool & 15) || ((uintptr_t)blk_pool & 15))
    return SI_ERR_ARG;
  if (G > 65535) return SI_ERR_TOO_LARGE;
  if (n_tokens == 0 || n_seqs == 0) return SI_OK;
  if (!blk_pool) P = 0;
  si::PlanesLayout tl{G, tok_rows, kd, vd}, bl{G, blk_rows > 0 ? blk_rows : 1, kd, vd};
#define SI_WPM_CASE(KD16, VD8)                                                                      \
  if (kd <= 16 * KD16 && vd <= 8 * VD8)                                                             \
    return launch_wp_attention_mma<KD16, VD8>(q, q_stride, positions, cu_q, n_seqs, tok_pool,       \
                                              tok_table, tok_table_stride, tl, blk_pool, blk_table, \
                                              blk_table_stride, bl, out, out_stride, n_tokens, H,   \
                                              scale, W, P, freq_v, key_splits, scratch, stream);
  SI_WPM_CASE(4, 8)
  SI_WPM_CASE(4, 16)
  SI_WPM_CASE(8, 16)
#undef SI_WPM_CASE
  return SI_ERR_UNSUPPORTED;
}
