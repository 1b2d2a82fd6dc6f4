// Multi-head attention over paged per-head keys and values, for decoders whose layers cache `row_width` elements per token:
//   columns of a token = [ ... keys of every key head (from k_off) ... | ... values of every value head (from v_off) ... ]
// Inside a block of `page` tokens the pool is head-group-major: the keys that one key/value head group needs of the block's tokens
// lie together (page x (maps * dim) elements), then the next group's, and after all keys the values likewise (page x vdim each), so
// a block reading one group's keys or values of consecutive tokens reads consecutive memory (head_slice_base below).
//
//   heads_prepare_kernel : from a token's projected (and, where the layer has one, convolved) row: RMS-norms every query head and
//                          key head over its `d` elements (optional weight), multiplies the queries by the position's temperature
//                          1 + coef * ln(floor((p + 1) / every) + 1), writes keys and values into the token's cache slot and the
//                          queries into a dense fp32 buffer.  A layer that reads another layer's cache passes no key / value columns.
//   paged_heads_attn_kernel : one block per (query token, key/value head): the query rows that share that head - `rep` query heads
//                          times `maps` soft-max maps (differential attention keeps two keys per head and one value) - each take a
//                          warp; key tiles of 32 rows pass through shared memory, fp32 online soft-max.  Optional learned bias per
//                          (distance bucket, head), added after the scale; optional sliding window.  Prompts, portions of prompts
//                          and decoded tokens are the same case: every key is read back from the cache.
//   paged_heads_attn_mma_kernel : the same on bfloat16 caches with m16n8k16 tensor-core products; one block per (sequence, key/value
//                          head, tile of query tokens), rows = (map, token, query head of the group); see the note above the kernel.
//   paged_heads_attn_dec_kernel : decode form of the tensor-core kernel for steps of few rows (see the note above the kernel).
//   diff_combine_kernel  : o = a1 - lambda a2 per head, o / sqrt(mean(o^2) + eps) * out_scale.
#include "seq_common.cuh"

#include <cstdlib>

namespace b200 {
namespace seq {

constexpr int kPrepThreads = 256;

// first element of token `tk` of block `block` in slice `slice` (w columns wide) of the column region that starts at column `off`
__device__ __forceinline__ int64_t head_slice_base(int64_t block, int tk, int page, int64_t RW, int off, int slice, int w) {
  return block * page * RW + (int64_t)off * page + (int64_t)slice * page * w + (int64_t)tk * w;
}

template <typename T>
__global__ void __launch_bounds__(kPrepThreads) heads_prepare_kernel(
    const float* __restrict__ src, int64_t ld, int col_q, int Hq, int d, const T* __restrict__ qnorm_w, float temp_coef, int temp_every,
    int col_k, int Hk, const T* __restrict__ knorm_w, int col_v, int Cv, int normalise, const int64_t* __restrict__ position_ids,
    const int64_t* __restrict__ slot_mapping, T* __restrict__ cache, int64_t RW, int k_off, int v_off, int page, int k_group, int v_w,
    float* __restrict__ q_out, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t t = blockIdx.x;
  const int w = warp_id(), lane = lane_id(), nw = kPrepThreads / 32;
  const int64_t pos = position_ids[t];
  const int64_t slot = slot_mapping[t];
  const float* row = src + t * ld;
  float temp = 1.f;
  if (temp_coef != 0.f && temp_every > 0) temp = 1.f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.f);
  const int n_heads = Hq + (col_k >= 0 ? Hk : 0);
  for (int hh = w; hh < n_heads; hh += nw) {
    const bool is_q = hh < Hq;
    const int h = is_q ? hh : hh - Hq;
    const float* v = row + (is_q ? col_q : col_k) + (int64_t)h * d;
    float rstd = 1.f;
    if (normalise) {
      float s = 0.f;
      for (int i = lane; i < d; i += 32) s += v[i] * v[i];
      rstd = 1.f / sqrtf(warp_sum(s) / d + eps);
    }
    const T* nw_ptr = is_q ? qnorm_w : knorm_w;
    if (is_q) {
      float* dst = q_out + (t * Hq + h) * d;
      for (int i = lane; i < d; i += 32) dst[i] = v[i] * rstd * (nw_ptr ? ldf(nw_ptr + i) : 1.f) * temp;
    } else if (slot >= 0) {
      T* dst = cache + head_slice_base(slot / page, (int)(slot % page), page, RW, k_off, h / k_group, k_group * d) + (h % k_group) * d;
      for (int i = lane; i < d; i += 32) stf(dst + i, v[i] * rstd * (nw_ptr ? ldf(nw_ptr + i) : 1.f));
    }
  }
  if (col_v >= 0 && slot >= 0) {
    for (int i = threadIdx.x; i < Cv; i += kPrepThreads)
      stf(cache + head_slice_base(slot / page, (int)(slot % page), page, RW, v_off, i / v_w, v_w) + i % v_w, row[col_v + i]);
  }
}

constexpr int kAttnWarps = 8, kKeyTile = 32;

// RPW query rows per warp, NV = ceil(dv / 32) value columns per lane
template <typename T, int RPW, int NV>
__global__ void __launch_bounds__(kAttnWarps * 32) paged_heads_attn_kernel(
    const float* __restrict__ q, const T* __restrict__ cache, int64_t RW, int k_off, int v_off, const int32_t* __restrict__ block_table,
    int64_t bt_stride, const int32_t* __restrict__ seq_of_token, const int64_t* __restrict__ position_ids, float* __restrict__ out, int H,
    int rep, int maps, int d, int dv, int window, float scale, int page, const float* __restrict__ rel, const int32_t* __restrict__ bucket_tab,
    int n_bucket_tab, int rel_rows) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  const int KD = maps * d, KP = KD + 1, rows_g = rep * maps, rows_blk = kAttnWarps * RPW;
  float* qs = sm;                       // [rows_blk][d]
  float* ks = qs + rows_blk * d;        // [kKeyTile][KP]
  float* vs = ks + kKeyTile * KP;       // [kKeyTile][dv]
  const int64_t t = blockIdx.x;
  const int g = blockIdx.y, r_base = blockIdx.z * rows_blk;
  const int w = warp_id(), lane = lane_id();
  const int Hq = H * maps;
  const int b = seq_of_token[t];
  const int p = (int)position_ids[t];
  const int j_lo = max(0, p - window + 1);
  const int nthreads = kAttnWarps * 32;
  // row r of the group: query head g * rep + r / maps, map r % maps
  for (int idx = threadIdx.x; idx < rows_blk * d; idx += nthreads) {
    const int r = r_base + idx / d;
    float v = 0.f;
    if (r < rows_g) {
      const int qh = (g * rep + r / maps) * maps + r % maps;
      v = q[(t * Hq + qh) * d + idx % d];
    }
    qs[idx] = v;
  }
  float m[RPW], l[RPW], acc[RPW][NV];
#pragma unroll
  for (int a = 0; a < RPW; ++a) {
    m[a] = -INFINITY;
    l[a] = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) acc[a][i] = 0.f;
  }
  const int32_t* table = block_table + (int64_t)b * bt_stride;
  for (int j0 = j_lo; j0 <= p; j0 += kKeyTile) {
    __syncthreads();
    const int nk = min(kKeyTile, p - j0 + 1);
    for (int idx = threadIdx.x; idx < nk * KD; idx += nthreads) {
      const int jj = idx / KD, dd = idx % KD;
      const int j = j0 + jj;
      ks[jj * KP + dd] = ldf(cache + head_slice_base(table[j / page], j % page, page, RW, k_off, g, KD) + dd);
    }
    for (int idx = threadIdx.x; idx < nk * dv; idx += nthreads) {
      const int jj = idx / dv, dd = idx % dv;
      const int j = j0 + jj;
      vs[jj * dv + dd] = ldf(cache + head_slice_base(table[j / page], j % page, page, RW, v_off, g, dv) + dd);
    }
    __syncthreads();
#pragma unroll
    for (int a = 0; a < RPW; ++a) {
      const int rl = w * RPW + a, r = r_base + rl;
      if (r >= rows_g) continue;  // warp-uniform
      const int mp = r % maps, h = g * rep + r / maps;
      float s = -INFINITY;
      if (lane < nk) {
        float dot = 0.f;
        const float* kq = ks + lane * KP + mp * d;
        const float* qq = qs + rl * d;
        for (int i = 0; i < d; ++i) dot = fmaf(qq[i], kq[i], dot);
        s = dot * scale;
        if (rel) {
          const int dist = p - (j0 + lane);
          const int bk = dist < n_bucket_tab ? bucket_tab[dist] : rel_rows - 1;
          s += rel[bk * H + h];
        }
      }
      const float m_new = fmaxf(m[a], warp_max(s));
      const float pr = lane < nk ? expf(s - m_new) : 0.f;
      const float corr = expf(m[a] - m_new);
      l[a] = l[a] * corr + warp_sum(pr);
      m[a] = m_new;
#pragma unroll
      for (int i = 0; i < NV; ++i) acc[a][i] *= corr;
      for (int jj = 0; jj < nk; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, pr, jj);
        const float* vr = vs + jj * dv;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int c = lane + 32 * i;
          if (c < dv) acc[a][i] = fmaf(pj, vr[c], acc[a][i]);
        }
      }
    }
  }
#pragma unroll
  for (int a = 0; a < RPW; ++a) {
    const int r = r_base + w * RPW + a;
    if (r >= rows_g) continue;
    const int qh = (g * rep + r / maps) * maps + r % maps;
    const float inv = 1.f / l[a];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < dv) out[(t * Hq + qh) * dv + c] = acc[a][i] * inv;
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------------
// Tensor-core form for bfloat16 caches.  One block of four warps per (sequence, key/value head, tile of query tokens): its 64
// rows are (map, token of the tile, query head of the group), map-major, so a warp's 16 rows share one map and read that map's
// key columns; both maps read the same value tile, which is loaded once.  Key / value tiles of KT rows come in with 16-byte
// cp.async, two stages deep; S = Q K^T and O += P V are m16n8k16 products, each warp keeps the running max, sum and output of
// its own rows in registers (no exchange between warps), P stays in registers between the two products.  Bias and masks are
// applied to S per element, so a tile may mix tokens at different positions.  Needs dim % 16 == 0, vdim % 16 == 0,
// vdim <= 256, (heads / kv_heads) * maps dividing 64 and 16-byte aligned head slices; everything else takes the plain kernel.
// ------------------------------------------------------------------------------------------------------------------------
constexpr int kMmaRows = 64, kMmaThreads = 128, kMmaPad = 8;

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int NDV, int KT, int STAGES>  // NDV = vdim / 8 output n-tiles per warp, KT keys per tile, STAGES tile buffers
__global__ void __launch_bounds__(kMmaThreads) paged_heads_attn_mma_kernel(
    const float* __restrict__ q, const __nv_bfloat16* __restrict__ cache, int64_t RW, int k_off, int v_off, const int32_t* __restrict__ block_table,
    int64_t bt_stride, const int32_t* __restrict__ cu_q, const int64_t* __restrict__ position_ids, float* __restrict__ out, int B, int H, int rep,
    int maps, int d, int window, float scale, int page, const float* __restrict__ rel, const int32_t* __restrict__ bucket_tab, int n_bucket_tab,
    int rel_rows, float* __restrict__ partial) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int dv = NDV * 8, VP = dv + kMmaPad;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int KD = maps * d, KP = KD + kMmaPad, DP = d + kMmaPad;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [64][DP]
  __nv_bfloat16* Ks = Qs + kMmaRows * DP;                            // [STAGES][KT][KP]
  __nv_bfloat16* Vs = Ks + STAGES * KT * KP;                         // [STAGES][KT][VP]
  const int rpm = kMmaRows / maps;   // rows per map
  const int QT = rpm / rep;          // query tokens per tile
  // which (sequence, tile of its tokens) this block has
  int tile = blockIdx.x, b = 0;
  for (; b < B; ++b) {
    const int nt = (cu_q[b + 1] - cu_q[b] + QT - 1) / QT;
    if (tile < nt) break;
    tile -= nt;
  }
  if (b >= B) return;  // block-uniform: no barrier has been met yet
  const int g = blockIdx.y;
  const int row0 = cu_q[b] + tile * QT;
  const int ntok = min(QT, cu_q[b + 1] - row0);
  const int p0 = (int)position_ids[row0], p_last = p0 + ntok - 1;
  // gridDim.z > 1: the tile's key tiles are dealt out in contiguous runs to gridDim.z blocks, whose (unnormalised output, max, sum)
  // per row are merged by paged_heads_attn_merge_kernel; a block whose run is empty records an empty partial
  const int j_first = max(0, p0 - window + 1);
  const int n_ktiles = (p_last - j_first + KT) / KT;
  const int per_split = (n_ktiles + gridDim.z - 1) / gridDim.z;
  const int j_start = j_first + (int)blockIdx.z * per_split * KT;
  const int j_end = min(p_last, j_start + per_split * KT - 1);   // last key of this block's run
  const int w = warp_id(), lane = lane_id();
  const int Hq = H * maps;
  const int32_t* table = block_table + (int64_t)b * bt_stride;
  for (int r = w; r < kMmaRows; r += kMmaThreads / 32) {  // one division set per row, not per element
    const int mp = r / rpm, rr = r % rpm, tok = rr / rep, hh = rr % rep;
    const float* src = q + ((int64_t)(row0 + tok) * Hq + (g * rep + hh) * maps + mp) * d;
    const bool live = tok < ntok;
    for (int c = lane; c < d; c += 32) Qs[r * DP + c] = __float2bfloat16_rn(live ? src[c] * scale : 0.f);
  }
  const int kchunks = KD / 8, vchunks = dv / 8, cpr = kchunks + vchunks;
  const int page_shift = (page & (page - 1)) == 0 ? 31 - __clz(page) : -1;
  // eight threads per key row: one block-table lookup per thread and row, then the row's 16-byte pieces go round the eight
  auto load_tile = [&](int stage, int j0) {
    __nv_bfloat16* kd = Ks + stage * KT * KP;
    __nv_bfloat16* vd = Vs + stage * KT * VP;
    for (int row = threadIdx.x >> 3; row < KT; row += kMmaThreads / 8) {
      const int j = j0 + row;
      __nv_bfloat16* krow = kd + row * KP;
      __nv_bfloat16* vrow = vd + row * VP;
      if (j <= j_end) {
        const int64_t blk = table[page_shift >= 0 ? j >> page_shift : j / page];
        const int tk = page_shift >= 0 ? j & (page - 1) : j % page;
        const __nv_bfloat16* ksrc = cache + head_slice_base(blk, tk, page, RW, k_off, g, KD);
        const __nv_bfloat16* vsrc = cache + head_slice_base(blk, tk, page, RW, v_off, g, dv);
        for (int ch = threadIdx.x & 7; ch < kchunks; ch += 8) cp_async_16(krow + ch * 8, ksrc + ch * 8, true);
        for (int ch = threadIdx.x & 7; ch < vchunks; ch += 8) cp_async_16(vrow + ch * 8, vsrc + ch * 8, true);
      } else {
        for (int ch = threadIdx.x & 7; ch < kchunks; ch += 8) *reinterpret_cast<uint4*>(krow + ch * 8) = make_uint4(0u, 0u, 0u, 0u);
        for (int ch = threadIdx.x & 7; ch < vchunks; ch += 8) *reinterpret_cast<uint4*>(vrow + ch * 8) = make_uint4(0u, 0u, 0u, 0u);  // finite: p = 0
      }
    }
    cp_async_commit();
  };
  // this thread's two accumulator rows
  const int cq = (lane & 3) * 2;
  int p_row[2], h_row[2];
  bool valid[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = w * 16 + (lane >> 2) + i * 8, rr = r % rpm, tok = rr / rep;
    valid[i] = tok < ntok;
    p_row[i] = valid[i] ? p0 + tok : p0;
    h_row[i] = g * rep + rr % rep;
  }
  const float rel_far[2] = {rel ? rel[(rel_rows - 1) * H + h_row[0]] : 0.f, rel ? rel[(rel_rows - 1) * H + h_row[1]] : 0.f};
  const int mp_w = (w * 16) / rpm;
  const bool warp_active = ((w * 16) % rpm) / rep < ntok;  // rows of a warp ascend in token: its first row decides
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[NDV][4];
#pragma unroll
  for (int i = 0; i < NDV; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const uint32_t qs_addr = smem_u32(Qs), ks_addr = smem_u32(Ks), vs_addr = smem_u32(Vs);
  const int lm = lane >> 3, lr = lane & 7;
  const uint32_t a_lane = qs_addr + (uint32_t)(((w * 16 + (lm & 1) * 8 + lr) * DP + (lm >> 1) * 8) * 2);
  // STAGES - 1 tiles are in flight ahead of the one being used; every iteration commits one group (an empty one past the end),
  // so "at most STAGES - 1 groups pending" always means that the current tile has landed
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    if (j_start + st * KT <= j_end) load_tile(st, j_start + st * KT);
    else cp_async_commit();
  }
  int stage = 0;
  for (int j0 = j_start; j0 <= j_end; j0 += KT, stage = stage + 1 == STAGES ? 0 : stage + 1) {
    {
      const int jn = j0 + (STAGES - 1) * KT;
      if (jn <= j_end) load_tile(stage == 0 ? STAGES - 1 : stage - 1, jn);
      else cp_async_commit();
      cp_async_wait<STAGES - 1>();
    }
    __syncthreads();  // the tile (and, first time round, Qs) is in shared memory
    if (warp_active) {
      float s[KT / 8][4];
#pragma unroll
      for (int i = 0; i < KT / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
      const uint32_t b_lane = ks_addr + (uint32_t)(((stage * KT + (lm >> 1) * 8 + lr) * KP + mp_w * d + (lm & 1) * 8) * 2);
      for (int kk = 0; kk < d; kk += 16) {
        uint32_t a[4];
        ldmatrix_x4(a[0], a[1], a[2], a[3], a_lane + kk * 2);
#pragma unroll
        for (int kg = 0; kg < KT / 16; ++kg) {
          uint32_t bb[4];
          ldmatrix_x4(bb[0], bb[1], bb[2], bb[3], b_lane + (uint32_t)((kg * 16 * KP + kk) * 2));
          mma_m16n8k16_bf16f32(s[2 * kg], a, bb[0], bb[1]);
          mma_m16n8k16_bf16f32(s[2 * kg + 1], a, bb[2], bb[3]);
        }
      }
      float mx[2] = {-INFINITY, -INFINITY};
      if (j0 + KT - 1 <= min(j_end, p0) && p_last - j0 < window && (!rel || p0 - (j0 + KT - 1) >= n_bucket_tab)) {
        // an interior tile: every key is visible to every row and (with a bias) lies in the last bucket
#pragma unroll
        for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            s[nt][e] += rel_far[e >> 1];
            mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
          }
      } else {
#pragma unroll
        for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = e >> 1, j = j0 + nt * 8 + cq + (e & 1);
            const int dist = p_row[i] - j;
            float v = s[nt][e];
            if (dist < 0 || dist >= window || j > j_end) {
              v = -INFINITY;
            } else if (rel) {
              v += rel[(dist < n_bucket_tab ? bucket_tab[dist] : rel_rows - 1) * H + h_row[i]];
            }
            s[nt][e] = v;
            mx[i] = fmaxf(mx[i], v);
          }
      }
      float m_use[2], corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
        const float m_new = fmaxf(m_run[i], mx[i]);
        m_use[i] = m_new == -INFINITY ? 0.f : m_new;  // a row that has met no visible key yet
        corr[i] = expf(m_run[i] - m_use[i]);
        m_run[i] = m_new;
      }
      uint32_t pa[KT / 16][4];
#pragma unroll
      for (int nt = 0; nt < KT / 8; ++nt) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(expf(s[nt][0] - m_use[0]), expf(s[nt][1] - m_use[0]));
        const __nv_bfloat162 hi = __floats2bfloat162_rn(expf(s[nt][2] - m_use[1]), expf(s[nt][3] - m_use[1]));
        // the sums use the rounded probabilities: numerator and denominator see the same weights
        sum[0] += __low2float(lo) + __high2float(lo);
        sum[1] += __low2float(hi) + __high2float(hi);
        pa[nt >> 1][(nt & 1) * 2] = *reinterpret_cast<const uint32_t*>(&lo);
        pa[nt >> 1][(nt & 1) * 2 + 1] = *reinterpret_cast<const uint32_t*>(&hi);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
        sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
        l_run[i] = l_run[i] * corr[i] + sum[i];
      }
#pragma unroll
      for (int i = 0; i < NDV; ++i) {
        o[i][0] *= corr[0];
        o[i][1] *= corr[0];
        o[i][2] *= corr[1];
        o[i][3] *= corr[1];
      }
      const uint32_t v_lane = vs_addr + (uint32_t)(((stage * KT + (lm & 1) * 8 + lr) * VP + (lm >> 1) * 8) * 2);
#pragma unroll
      for (int kg = 0; kg < KT / 16; ++kg) {
#pragma unroll
        for (int nt = 0; nt < NDV; nt += 2) {
          uint32_t bb[4];
          ldmatrix_x4_trans(bb[0], bb[1], bb[2], bb[3], v_lane + (uint32_t)((kg * 16 * VP + nt * 8) * 2));
          mma_m16n8k16_bf16f32(o[nt], pa[kg], bb[0], bb[1]);
          mma_m16n8k16_bf16f32(o[nt + 1], pa[kg], bb[2], bb[3]);
        }
      }
    }
    __syncthreads();  // everyone is done with this stage before the next iteration's load overwrites it
  }
  if (gridDim.z > 1) {
    // partial [tile][g][split][64 rows][dv + 2]: unnormalised output, then the running max and sum
    float* base = partial + ((((int64_t)blockIdx.x * gridDim.y + g) * gridDim.z + blockIdx.z) * kMmaRows) * (dv + 2);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (!valid[i]) continue;
      float* dst = base + (int64_t)(w * 16 + (lane >> 2) + i * 8) * (dv + 2);
#pragma unroll
      for (int nt = 0; nt < NDV; ++nt) {
        dst[nt * 8 + cq] = o[nt][i * 2];
        dst[nt * 8 + cq + 1] = o[nt][i * 2 + 1];
      }
      if ((lane & 3) == 0) {
        dst[dv] = m_run[i];
        dst[dv + 1] = l_run[i];
      }
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (!valid[i]) continue;
    const int r = w * 16 + (lane >> 2) + i * 8, rr = r % rpm;
    const int qh = (g * rep + rr % rep) * maps + r / rpm;
    float* dst = out + ((int64_t)(row0 + rr / rep) * Hq + qh) * dv;
    const float inv = 1.f / l_run[i];
#pragma unroll
    for (int nt = 0; nt < NDV; ++nt) {
      dst[nt * 8 + cq] = o[nt][i * 2] * inv;
      dst[nt * 8 + cq + 1] = o[nt][i * 2 + 1] * inv;
    }
  }
}

// out[row] = sum_z e^(m_z - M) O_z / sum_z e^(m_z - M) l_z over the key splits of paged_heads_attn_mma_kernel; one block per
// (query tile, key/value head), one warp per row
__global__ void __launch_bounds__(256) paged_heads_attn_merge_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                                                    const int32_t* __restrict__ cu_q, int B, int H, int rep, int maps, int dv,
                                                                    int nsplit) {
  pdl_launch_dependents();
  pdl_wait();
  const int rpm = kMmaRows / maps, QT = rpm / rep;
  int tile = blockIdx.x, b = 0;
  for (; b < B; ++b) {
    const int nt = (cu_q[b + 1] - cu_q[b] + QT - 1) / QT;
    if (tile < nt) break;
    tile -= nt;
  }
  if (b >= B) return;
  const int g = blockIdx.y, lane = lane_id();
  const int row0 = cu_q[b] + tile * QT;
  const int ntok = min(QT, cu_q[b + 1] - row0);
  const int Hq = H * maps;
  constexpr int kMaxSplit = 8;
  for (int r = warp_id(); r < kMmaRows; r += 8) {
    const int rr = r % rpm, tok = rr / rep;
    if (tok >= ntok) continue;
    const float* base = partial + ((((int64_t)blockIdx.x * gridDim.y + g) * nsplit) * kMmaRows + r) * (dv + 2);
    const int64_t zs = (int64_t)kMmaRows * (dv + 2);
    float M = -INFINITY, wz[kMaxSplit];
#pragma unroll
    for (int z = 0; z < kMaxSplit; ++z) {
      wz[z] = z < nsplit ? base[z * zs + dv] : -INFINITY;
      M = fmaxf(M, wz[z]);
    }
    float den = 0.f;
#pragma unroll
    for (int z = 0; z < kMaxSplit; ++z) {
      wz[z] = wz[z] > -INFINITY ? expf(wz[z] - M) : 0.f;  // an empty run carries no weight
      if (z < nsplit) den += wz[z] * base[z * zs + dv + 1];
    }
    const float inv = 1.f / den;
    float* dst = out + ((int64_t)(row0 + tok) * Hq + (g * rep + rr % rep) * maps + r / rpm) * dv;
    for (int c = lane; c < dv; c += 32) {
      float acc = 0.f;
#pragma unroll
      for (int z = 0; z < kMaxSplit; ++z)
        if (z < nsplit) acc = fmaf(wz[z], base[z * zs + c], acc);
      dst[c] = acc * inv;
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------------
// Decode form of the tensor-core kernel, for steps of few query rows.  One block of four warps per (query token, key/value head,
// run of the token's keys): the token's rows of that head group - (rep query heads) x maps, at most 16 - are ONE m16 tile; rows
// 0..7 carry map 1 and rows 8..15 map 2 when there are two maps.  Every warp scores the whole 16-key tile (the same S in all four:
// a few MMAs) and keeps the same running max and sum, but accumulates only its quarter of the value columns, so a thread holds
// vdim / 16 output values instead of vdim / 2 and several blocks share an SM, each with three small tiles in flight: the
// key / value stream of a decoding step is bound by memory latency, not by work.  Partials per run are merged by
// paged_heads_attn_dec_merge_kernel.  Needs dim % 16 == 0, vdim % 64 == 0, rep * maps <= 16 (rep <= 8 with two maps).
// ------------------------------------------------------------------------------------------------------------------------
constexpr int kDecKT = 16, kDecStages = 4, kDecRows = 16;

template <int NDVW>  // n-tiles (8 value columns each) per warp: vdim = 32 * NDVW
__global__ void __launch_bounds__(kMmaThreads) paged_heads_attn_dec_kernel(
    const float* __restrict__ q, const __nv_bfloat16* __restrict__ cache, int64_t RW, int k_off, int v_off, const int32_t* __restrict__ block_table,
    int64_t bt_stride, const int32_t* __restrict__ seq_of_token, const int64_t* __restrict__ position_ids, float* __restrict__ out, int H, int rep,
    int maps, int d, int window, float scale, int page, const float* __restrict__ rel, const int32_t* __restrict__ bucket_tab, int n_bucket_tab,
    int rel_rows, float* __restrict__ partial) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int dv = NDVW * 32, VP = dv + kMmaPad, KT = kDecKT, STAGES = kDecStages;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int KD = maps * d, KP = KD + kMmaPad, DP = d + kMmaPad;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [16][DP]
  __nv_bfloat16* Ks = Qs + kDecRows * DP;                            // [STAGES][KT][KP]
  __nv_bfloat16* Vs = Ks + STAGES * KT * KP;                         // [STAGES][KT][VP]
  const int64_t t = blockIdx.x;
  const int g = blockIdx.y;
  const int b = seq_of_token[t];
  const int p = (int)position_ids[t];
  const int j_first = max(0, p - window + 1);
  const int n_ktiles = (p - j_first + KT) / KT;
  const int per_split = (n_ktiles + gridDim.z - 1) / gridDim.z;
  const int j_start = j_first + (int)blockIdx.z * per_split * KT;
  const int j_end = min(p, j_start + per_split * KT - 1);
  const int w = warp_id(), lane = lane_id();
  const int Hq = H * maps;
  const int32_t* table = block_table + (int64_t)b * bt_stride;
  // row r of the tile: two maps -> map r / 8, head r % 8 of the group; one map -> head r
  for (int r = w; r < kDecRows; r += kMmaThreads / 32) {
    const int mp = maps == 2 ? r >> 3 : 0, hh = maps == 2 ? r & 7 : r;
    const bool live = hh < rep;
    const float* src = q + ((int64_t)t * Hq + (g * rep + (live ? hh : 0)) * maps + mp) * d;
    for (int c = lane; c < d; c += 32) Qs[r * DP + c] = __float2bfloat16_rn(live ? src[c] * scale : 0.f);
  }
  const int kchunks = KD / 8, vchunks = dv / 8;
  const int page_shift = (page & (page - 1)) == 0 ? 31 - __clz(page) : -1;
  auto load_tile = [&](int stage, int j0) {  // eight threads per key row, sixteen rows: one pass
    const int row = threadIdx.x >> 3, j = j0 + row;
    __nv_bfloat16* krow = Ks + (stage * KT + row) * KP;
    __nv_bfloat16* vrow = Vs + (stage * KT + row) * VP;
    if (j <= j_end) {
      const int64_t blk = table[page_shift >= 0 ? j >> page_shift : j / page];
      const int tk = page_shift >= 0 ? j & (page - 1) : j % page;
      const __nv_bfloat16* ksrc = cache + head_slice_base(blk, tk, page, RW, k_off, g, KD);
      const __nv_bfloat16* vsrc = cache + head_slice_base(blk, tk, page, RW, v_off, g, dv);
      for (int ch = threadIdx.x & 7; ch < kchunks; ch += 8) cp_async_16(krow + ch * 8, ksrc + ch * 8, true);
      for (int ch = threadIdx.x & 7; ch < vchunks; ch += 8) cp_async_16(vrow + ch * 8, vsrc + ch * 8, true);
    } else {
      for (int ch = threadIdx.x & 7; ch < kchunks; ch += 8) *reinterpret_cast<uint4*>(krow + ch * 8) = make_uint4(0u, 0u, 0u, 0u);
      for (int ch = threadIdx.x & 7; ch < vchunks; ch += 8) *reinterpret_cast<uint4*>(vrow + ch * 8) = make_uint4(0u, 0u, 0u, 0u);  // finite: p = 0
    }
    cp_async_commit();
  };
  const int cq = (lane & 3) * 2;
  int h_row[2];
  bool valid[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = (lane >> 2) + i * 8, hh = maps == 2 ? r & 7 : r;
    valid[i] = hh < rep;
    h_row[i] = g * rep + (valid[i] ? hh : 0);
  }
  const float rel_far[2] = {rel ? rel[(rel_rows - 1) * H + h_row[0]] : 0.f, rel ? rel[(rel_rows - 1) * H + h_row[1]] : 0.f};
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[NDVW][4];
#pragma unroll
  for (int i = 0; i < NDVW; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const uint32_t qs_addr = smem_u32(Qs), ks_addr = smem_u32(Ks), vs_addr = smem_u32(Vs);
  const int lm = lane >> 3, lr = lane & 7;
  const uint32_t a_lane = qs_addr + (uint32_t)((((lm & 1) * 8 + lr) * DP + (lm >> 1) * 8) * 2);
  // STAGES - 1 tiles are in flight ahead of the one being used; every iteration commits one group (an empty one past the end),
  // so "at most STAGES - 1 groups pending" always means that the current tile has landed
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    if (j_start + st * KT <= j_end) load_tile(st, j_start + st * KT);
    else cp_async_commit();
  }
  int stage = 0;
  for (int j0 = j_start; j0 <= j_end; j0 += KT, stage = stage + 1 == STAGES ? 0 : stage + 1) {
    {
      const int jn = j0 + (STAGES - 1) * KT;
      if (jn <= j_end) load_tile(stage == 0 ? STAGES - 1 : stage - 1, jn);
      else cp_async_commit();
      cp_async_wait<STAGES - 1>();
    }
    __syncthreads();  // the tile (and, first time round, Qs) is in shared memory
    // the score products: even and odd k steps accumulate apart (two short chains of dependent MMAs instead of one long one)
    float s[2][4] = {}, s2[2][4] = {}, t1[2][4] = {}, t2[2][4] = {};
    const uint32_t b_lane = ks_addr + (uint32_t)(((stage * KT + (lm >> 1) * 8 + lr) * KP + (lm & 1) * 8) * 2);
#pragma unroll 2
    for (int kk = 0; kk < d; kk += 32) {
      uint32_t a[4], bb[4], a2[4], b2[4];
      const bool odd = kk + 16 < d;
      ldmatrix_x4(a[0], a[1], a[2], a[3], a_lane + kk * 2);
      ldmatrix_x4(bb[0], bb[1], bb[2], bb[3], b_lane + (uint32_t)(kk * 2));
      if (odd) {
        ldmatrix_x4(a2[0], a2[1], a2[2], a2[3], a_lane + (kk + 16) * 2);
        ldmatrix_x4(b2[0], b2[1], b2[2], b2[3], b_lane + (uint32_t)((kk + 16) * 2));
      }
      mma_m16n8k16_bf16f32(s[0], a, bb[0], bb[1]);
      mma_m16n8k16_bf16f32(s[1], a, bb[2], bb[3]);
      if (odd) {
        mma_m16n8k16_bf16f32(t1[0], a2, b2[0], b2[1]);
        mma_m16n8k16_bf16f32(t1[1], a2, b2[2], b2[3]);
      }
      if (maps == 2) {  // the second map's key columns; its rows are 8..15 of the tile
        ldmatrix_x4(bb[0], bb[1], bb[2], bb[3], b_lane + (uint32_t)((d + kk) * 2));
        if (odd) ldmatrix_x4(b2[0], b2[1], b2[2], b2[3], b_lane + (uint32_t)((d + kk + 16) * 2));
        mma_m16n8k16_bf16f32(s2[0], a, bb[0], bb[1]);
        mma_m16n8k16_bf16f32(s2[1], a, bb[2], bb[3]);
        if (odd) {
          mma_m16n8k16_bf16f32(t2[0], a2, b2[0], b2[1]);
          mma_m16n8k16_bf16f32(t2[1], a2, b2[2], b2[3]);
        }
      }
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      s[nt][0] += t1[nt][0];
      s[nt][1] += t1[nt][1];
      s[nt][2] = maps == 2 ? s2[nt][2] + t2[nt][2] : s[nt][2] + t1[nt][2];
      s[nt][3] = maps == 2 ? s2[nt][3] + t2[nt][3] : s[nt][3] + t1[nt][3];
    }
    float mx[2] = {-INFINITY, -INFINITY};
    if (j0 + KT - 1 <= j_end && p - j0 < window && (!rel || p - (j0 + KT - 1) >= n_bucket_tab)) {
      // an interior tile: every key is visible and (with a bias) lies in the last bucket - no per-element mask or lookup
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[nt][e] += rel_far[e >> 1];
          mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
        }
    } else {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = e >> 1, j = j0 + nt * 8 + cq + (e & 1);
          const int dist = p - j;
          float v = s[nt][e];
          if (dist < 0 || dist >= window || j > j_end) {
            v = -INFINITY;
          } else if (rel) {
            v += rel[(dist < n_bucket_tab ? bucket_tab[dist] : rel_rows - 1) * H + h_row[i]];
          }
          s[nt][e] = v;
          mx[i] = fmaxf(mx[i], v);
        }
    }
    float m_use[2], corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
      const float m_new = fmaxf(m_run[i], mx[i]);
      m_use[i] = m_new == -INFINITY ? 0.f : m_new;
      corr[i] = expf(m_run[i] - m_use[i]);
      m_run[i] = m_new;
    }
    uint32_t pa[4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(expf(s[nt][0] - m_use[0]), expf(s[nt][1] - m_use[0]));
      const __nv_bfloat162 hi = __floats2bfloat162_rn(expf(s[nt][2] - m_use[1]), expf(s[nt][3] - m_use[1]));
      sum[0] += __low2float(lo) + __high2float(lo);   // the rounded probabilities: numerator and denominator see the same weights
      sum[1] += __low2float(hi) + __high2float(hi);
      pa[nt * 2] = *reinterpret_cast<const uint32_t*>(&lo);
      pa[nt * 2 + 1] = *reinterpret_cast<const uint32_t*>(&hi);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
      sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
      l_run[i] = l_run[i] * corr[i] + sum[i];
    }
    if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {  // the running maxima settle after the first tiles
#pragma unroll
      for (int i = 0; i < NDVW; ++i) {
        o[i][0] *= corr[0];
        o[i][1] *= corr[0];
        o[i][2] *= corr[1];
        o[i][3] *= corr[1];
      }
    }
    const uint32_t v_lane = vs_addr + (uint32_t)(((stage * KT + (lm & 1) * 8 + lr) * VP + w * NDVW * 8 + (lm >> 1) * 8) * 2);
#pragma unroll
    for (int nt = 0; nt < NDVW; nt += 2) {
      uint32_t bb[4];
      ldmatrix_x4_trans(bb[0], bb[1], bb[2], bb[3], v_lane + (uint32_t)(nt * 8 * 2));
      mma_m16n8k16_bf16f32(o[nt], pa, bb[0], bb[1]);
      mma_m16n8k16_bf16f32(o[nt + 1], pa, bb[2], bb[3]);
    }
    __syncthreads();  // everyone is done with this stage before the next iteration's load overwrites it
  }
  // partial [token][g][split][16 rows][dv + 2]: unnormalised output, then the running max and sum (written by warp 0)
  float* base = partial + ((((int64_t)t * gridDim.y + g) * gridDim.z + blockIdx.z) * kDecRows) * (dv + 2);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (!valid[i]) continue;
    float* dst = base + (int64_t)((lane >> 2) + i * 8) * (dv + 2);
#pragma unroll
    for (int nt = 0; nt < NDVW; ++nt) {
      dst[(w * NDVW + nt) * 8 + cq] = o[nt][i * 2];
      dst[(w * NDVW + nt) * 8 + cq + 1] = o[nt][i * 2 + 1];
    }
    if (w == 0 && (lane & 3) == 0) {
      dst[dv] = m_run[i];
      dst[dv + 1] = l_run[i];
    }
  }
}

// one block per (token, key/value head), one warp per row of the 16-row tile (rows beyond the group's are skipped)
__global__ void __launch_bounds__(128) paged_heads_attn_dec_merge_kernel(const float* __restrict__ partial, float* __restrict__ out, int H, int rep,
                                                                        int maps, int dv, int nsplit) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t t = blockIdx.x;
  const int g = blockIdx.y, lane = lane_id(), Hq = H * maps;
  constexpr int kMaxSplit = 8;
  for (int r = warp_id(); r < kDecRows; r += 4) {
    const int mp = maps == 2 ? r >> 3 : 0, hh = maps == 2 ? r & 7 : r;
    if (hh >= rep) continue;
    const float* base = partial + ((((int64_t)t * gridDim.y + g) * nsplit) * kDecRows + r) * (dv + 2);
    const int64_t zs = (int64_t)kDecRows * (dv + 2);
    float M = -INFINITY, wz[kMaxSplit];
#pragma unroll
    for (int z = 0; z < kMaxSplit; ++z) {
      wz[z] = z < nsplit ? base[z * zs + dv] : -INFINITY;
      M = fmaxf(M, wz[z]);
    }
    float den = 0.f;
#pragma unroll
    for (int z = 0; z < kMaxSplit; ++z) {
      wz[z] = wz[z] > -INFINITY ? expf(wz[z] - M) : 0.f;  // an empty run carries no weight
      if (z < nsplit) den += wz[z] * base[z * zs + dv + 1];
    }
    const float inv = 1.f / den;
    float* dst = out + ((int64_t)t * Hq + (g * rep + hh) * maps + mp) * dv;
    for (int c = lane; c < dv; c += 32) {
      float acc = 0.f;
#pragma unroll
      for (int z = 0; z < kMaxSplit; ++z)
        if (z < nsplit) acc = fmaf(wz[z], base[z * zs + c], acc);
      dst[c] = acc * inv;
    }
  }
}

// in [T, H, 2, dv] fp32 (two maps per head) -> out [T, H * dv]: o = a1 - lambda a2, unit RMS over dv, times out_scale
template <typename TO>
__global__ void __launch_bounds__(256) diff_combine_kernel(const float* __restrict__ in, TO* __restrict__ out, int H, int dv, float lambda,
                                                           float out_scale, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t t = blockIdx.x;
  const int lane = lane_id();
  for (int h = warp_id(); h < H; h += 8) {
    const float* a1 = in + ((t * H + h) * 2) * dv;
    const float* a2 = a1 + dv;
    float s = 0.f;
    for (int i = lane; i < dv; i += 32) {
      const float o = a1[i] - lambda * a2[i];
      s += o * o;
    }
    const float rstd = 1.f / sqrtf(warp_sum(s) / dv + eps);
    for (int i = lane; i < dv; i += 32) stf(out + (t * H + h) * dv + i, (a1[i] - lambda * a2[i]) * rstd * out_scale);
  }
}

}  // namespace seq
}  // namespace b200

using namespace b200::seq;

// src: fp32 rows (leading dimension ld) holding Hq query heads of d elements from col_q, Hk key heads from col_k (col_k < 0: the
// layer writes no keys), Cv value elements from col_v (col_v < 0: no values).  normalise != 0: unit RMS over d per head (eps), times
// the weight when given.  Queries are multiplied by 1 + temp_coef ln(floor((p + 1) / temp_every) + 1) (temp_coef 0: by 1).
// The pool is written head-group-major inside a block of `page` tokens: k_group key heads and v_width value columns per group.
extern "C" int b200_seq_heads_prepare(const float* src, int64_t ld, int col_q, int Hq, int d, const void* qnorm_w, float temp_coef,
                                      int temp_every, int col_k, int Hk, const void* knorm_w, int col_v, int Cv, int normalise,
                                      const int64_t* position_ids, const int64_t* slot_mapping, void* cache, int dt, int64_t row_width,
                                      int k_off, int v_off, int page, int k_group, int v_width, float* q_out, int64_t T, float eps,
                                      void* stream) {
  if (T == 0) return B200_OK;
  if (Hq <= 0 || d <= 0 || page <= 0 || (col_k >= 0 && (k_group <= 0 || Hk % k_group != 0)) || (col_v >= 0 && (v_width <= 0 || Cv % v_width != 0))) {
    b200_set_last_error("seq_heads_prepare: bad sizes");
    return B200_ERR_ARG;
  }
  B200_SEQ_DISPATCH(dt, E, B200_LAUNCH((heads_prepare_kernel<E>), dim3((unsigned)T), dim3(kPrepThreads), 0, (cudaStream_t)stream, src, ld, col_q, Hq,
                                       d, (const E*)qnorm_w, temp_coef, temp_every, col_k, Hk, (const E*)knorm_w, col_v, Cv, normalise,
                                       position_ids, slot_mapping, (E*)cache, row_width, k_off, v_off, page, k_group > 0 ? k_group : 1,
                                       v_width > 0 ? v_width : 1, q_out, eps));
  b200_count_launches(1);
  return B200_OK;
}

template <typename T, int RPW, int NV>
static int launch_paged_heads_attn(const float* q, const void* cache, int64_t RW, int k_off, int v_off, const int32_t* block_table,
                                   int64_t bt_stride, const int32_t* seq_of_token, const int64_t* position_ids, float* out, int64_t Tq, int H,
                                   int G, int maps, int d, int dv, int window, float scale, int page, const float* rel,
                                   const int32_t* bucket_tab, int n_bucket_tab, int rel_rows, cudaStream_t st) {
  const int rep = H / G, rows_g = rep * maps, rows_blk = kAttnWarps * RPW;
  const size_t smem = ((size_t)rows_blk * d + (size_t)kKeyTile * (maps * d + 1) + (size_t)kKeyTile * dv) * 4;
  if (smem > 200 * 1024) { b200_set_last_error("seq_paged_attn: heads too wide"); return B200_ERR_ARG; }
  static bool cfg = false;
  if (!cfg) { cudaFuncSetAttribute(paged_heads_attn_kernel<T, RPW, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); cfg = true; }
  dim3 grid((unsigned)Tq, (unsigned)G, (unsigned)((rows_g + rows_blk - 1) / rows_blk));
  B200_LAUNCH((paged_heads_attn_kernel<T, RPW, NV>), grid, dim3(kAttnWarps * 32), smem, st, q, (const T*)cache, RW, k_off, v_off, block_table,
              bt_stride, seq_of_token, position_ids, out, H, rep, maps, d, dv, window, scale, page, rel, bucket_tab, n_bucket_tab, rel_rows);
  b200_count_launches(1);
  return B200_OK;
}

static bool attn_mma_shape_ok(int dt, int H, int G, int maps, int d, int dv) {
  static const bool use_mma = []() { const char* e = getenv("B200_SEQ_ATTN_MMA"); return !(e && e[0] == '0'); }();
  return use_mma && dt == B200_DT_BF16 && G > 0 && H % G == 0 && maps >= 1 && maps <= 2 && kMmaRows % ((H / G) * maps) == 0 && d % 16 == 0 &&
         dv % 16 == 0 && dv <= 256;
}

// steps of few rows whose head group fits one m16 tile take the decode form
static bool attn_dec_ok(int dt, int64_t Tq, int H, int G, int maps, int d, int dv) {
  if (!attn_mma_shape_ok(dt, H, G, maps, d, dv)) return false;
  const int rep = H / G;
  return dv % 64 == 0 && (maps == 2 ? rep <= 8 : rep <= 16) && Tq * G < 2 * 148;
}

// Over how many blocks the tensor-core kernels should split a query tile's keys for this step (1: no split; 0: the shape takes the
// plain kernel) and the fp32 workspace (`partial`) that takes: steps with few query rows (decoding) would leave most SMs idle with one
// block per (query tile, key/value head).
extern "C" int b200_seq_paged_attn_splits(int dt, int64_t Tq, int B, int H, int G, int maps, int d, int dv, int64_t* workspace_floats) {
  if (workspace_floats) *workspace_floats = 0;
  if (!attn_mma_shape_ok(dt, H, G, maps, d, dv)) return 0;
  if (attn_dec_ok(dt, Tq, H, G, maps, d, dv)) {
    // as many runs as keep all blocks resident at once (shared memory decides how many share an SM): a second, thinner wave of
    // blocks would double the time of a step that is bound by latency
    const int64_t smem = ((int64_t)kDecRows * (d + kMmaPad) + (int64_t)kDecStages * kDecKT * ((maps * d + kMmaPad) + (dv + kMmaPad))) * 2 + 1024;
    int64_t per_sm = (220 * 1024) / smem;
    per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
    int64_t n = (148 * per_sm) / (Tq * G);
    n = n < 2 ? 2 : (n > 8 ? 8 : n);
    if (workspace_floats) *workspace_floats = Tq * G * n * kDecRows * (dv + 2);
    return (int)n;
  }
  const int QT = kMmaRows / ((H / G) * maps);
  const int64_t tiles = (Tq + QT - 1) / QT + B;
  const int64_t busy = ((Tq + QT - 1) / QT > B ? (Tq + QT - 1) / QT : B) * G;   // blocks that have rows: between the two bounds
  int64_t n = (2 * 148) / (busy > 0 ? busy : 1);
  n = n < 1 ? 1 : (n > 8 ? 8 : n);
  if (n > 1 && workspace_floats) *workspace_floats = tiles * G * n * kMmaRows * (dv + 2);
  return (int)n;
}

// q fp32 [Tq, H * maps, d] (query head h, map m at index h * maps + m); cache [blocks, page, row_width] of type dt with G * maps key
// heads of d elements from k_off (key head g, map m at g * maps + m) and G value heads of dv elements from v_off; out fp32
// [Tq, H * maps, dv].  window <= 0: every earlier token is visible.  rel (fp32 [rel_rows, H]) NULL: no bias; otherwise
// rel[bucket(distance), h] is added to the scaled score, bucket(n) = bucket_tab[n] for n < n_bucket_tab and rel_rows - 1 beyond.
// cu_q [B + 1]: row boundaries of the step's sequences (the tensor-core kernel tiles a sequence's rows; NULL: plain kernel only).
// `partial` / nsplit: from b200_seq_paged_attn_splits (NULL / <= 1: no split).
extern "C" int b200_seq_paged_attn(const float* q, const void* cache, int dt, int64_t row_width, int k_off, int v_off,
                                   const int32_t* block_table, int64_t bt_stride, const int32_t* seq_of_token, const int32_t* cu_q, int B,
                                   const int64_t* position_ids, float* out, int64_t Tq, int H, int G, int maps, int d, int dv, int window,
                                   float scale, int page, const float* rel, const int32_t* bucket_tab, int n_bucket_tab, int rel_rows,
                                   float* partial, int nsplit, void* stream) {
  if (Tq == 0) return B200_OK;
  if (G <= 0 || H % G != 0 || maps < 1 || d <= 0 || dv <= 0 || dv > 512) {
    b200_set_last_error("seq_paged_attn: need heads % kv_heads == 0, maps >= 1, 0 < vdim <= 512");
    return B200_ERR_ARG;
  }
  if (window <= 0) window = 0x3fffffff;
  cudaStream_t st = (cudaStream_t)stream;
  const int rows_g = (H / G) * maps;
  const bool aligned = row_width % 8 == 0 && k_off % 8 == 0 && v_off % 8 == 0 && (reinterpret_cast<uintptr_t>(cache) & 15) == 0;
  if (aligned && partial != nullptr && nsplit >= 2 && nsplit <= 8 && attn_dec_ok(dt, Tq, H, G, maps, d, dv)) {
    const size_t smem = ((size_t)kDecRows * (d + kMmaPad) + (size_t)kDecStages * kDecKT * ((maps * d + kMmaPad) + (dv + kMmaPad))) * 2;
    if (smem <= 200 * 1024) {
      dim3 grid((unsigned)Tq, (unsigned)G, (unsigned)nsplit);
#define PAD(N)                                                                                                                           \
  do {                                                                                                                                   \
    static bool cfg = false;                                                                                                             \
    if (!cfg) { cudaFuncSetAttribute(paged_heads_attn_dec_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); cfg = true; } \
    B200_LAUNCH((paged_heads_attn_dec_kernel<N>), grid, dim3(kMmaThreads), smem, st, q, (const __nv_bfloat16*)cache, row_width, k_off, v_off, \
                block_table, bt_stride, seq_of_token, position_ids, out, H, H / G, maps, d, window, scale, page, rel, bucket_tab,         \
                n_bucket_tab, rel_rows, partial);                                                                                        \
    B200_LAUNCH(paged_heads_attn_dec_merge_kernel, dim3((unsigned)Tq, (unsigned)G), dim3(128), 0, st, (const float*)partial, out, H, H / G, \
                maps, dv, nsplit);                                                                                                       \
    b200_count_launches(2);                                                                                                              \
    return B200_OK;                                                                                                                      \
  } while (0)
      switch (dv / 32) {
        case 2: PAD(2);
        case 4: PAD(4);
        case 6: PAD(6);
        case 8: PAD(8);
        default: break;
      }
#undef PAD
    }
  }
  if (attn_mma_shape_ok(dt, H, G, maps, d, dv) && cu_q != nullptr && row_width % 8 == 0 && k_off % 8 == 0 && v_off % 8 == 0 &&
      (reinterpret_cast<uintptr_t>(cache) & 15) == 0) {
    const int QT = kMmaRows / rows_g;
    const int64_t tiles = (Tq + QT - 1) / QT + B;  // upper bound of sum_b ceil(n_b / QT); surplus blocks return at once
    const int kt = dv <= 128 ? 64 : 32;
    const size_t stage_bytes = ((size_t)kt * (maps * d + kMmaPad) + (size_t)kt * (dv + kMmaPad)) * 2, q_bytes = (size_t)kMmaRows * (d + kMmaPad) * 2;
    if (!partial || nsplit < 1) nsplit = 1;
    if (nsplit > 8) nsplit = 8;
    // two tile buffers: measured on B200 at 32 sequences x 1040 keys, five buffers (one block per SM instead of two) ran the
    // split decode step 1.4x slower than two; the pipeline itself is written for any depth
    constexpr int stages = 2;
    const size_t smem = q_bytes + stages * stage_bytes;
    if (smem <= 200 * 1024 && tiles <= 0x7fffffff) {
      dim3 grid((unsigned)tiles, (unsigned)G, (unsigned)nsplit);
#define PAM_S(N, KT, S)                                                                                                                  \
  do {                                                                                                                                   \
    static bool cfg = false;                                                                                                             \
    if (!cfg) { cudaFuncSetAttribute(paged_heads_attn_mma_kernel<N, KT, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); cfg = true; } \
    B200_LAUNCH((paged_heads_attn_mma_kernel<N, KT, S>), grid, dim3(kMmaThreads), smem, st, q, (const __nv_bfloat16*)cache, row_width, k_off,  \
                v_off, block_table, bt_stride, cu_q, position_ids, out, B, H, H / G, maps, d, window, scale, page, rel, bucket_tab,         \
                n_bucket_tab, rel_rows, partial);                                                                                        \
    if (nsplit > 1)                                                                                                                      \
      B200_LAUNCH(paged_heads_attn_merge_kernel, dim3((unsigned)tiles, (unsigned)G), dim3(256), 0, st, (const float*)partial, out, cu_q, B, H, \
                  H / G, maps, dv, nsplit);                                                                                              \
    b200_count_launches(nsplit > 1 ? 2 : 1);                                                                                             \
    return B200_OK;                                                                                                                      \
  } while (0)
#define PAM(N, KT) PAM_S(N, KT, stages)
      switch (dv / 8) {
        case 2: PAM(2, 64);
        case 4: PAM(4, 64);
        case 6: PAM(6, 64);
        case 8: PAM(8, 64);
        case 10: PAM(10, 64);
        case 12: PAM(12, 64);
        case 14: PAM(14, 64);
        case 16: PAM(16, 64);
        case 18: PAM(18, 32);
        case 20: PAM(20, 32);
        case 22: PAM(22, 32);
        case 24: PAM(24, 32);
        case 26: PAM(26, 32);
        case 28: PAM(28, 32);
        case 30: PAM(30, 32);
        case 32: PAM(32, 32);
        default: break;
      }
#undef PAM_S
#undef PAM
    }
  }
  const int nv = (dv + 31) / 32;
#define PA(RPW, NV)                                                                                                                      \
  B200_SEQ_DISPATCH(dt, E, return (launch_paged_heads_attn<E, RPW, NV>(q, cache, row_width, k_off, v_off, block_table, bt_stride, seq_of_token, \
                                                                       position_ids, out, Tq, H, G, maps, d, dv, window, scale, page, rel,  \
                                                                       bucket_tab, n_bucket_tab, rel_rows, st)))
#define PA_NV(RPW)            \
  do {                        \
    if (nv <= 2) PA(RPW, 2);  \
    else if (nv <= 4) PA(RPW, 4); \
    else if (nv <= 8) PA(RPW, 8); \
    else PA(RPW, 16);         \
  } while (0)
  if (rows_g <= kAttnWarps) PA_NV(1);
  else PA_NV(2);
#undef PA_NV
#undef PA
  return B200_ERR_UNSUPPORTED;
}

extern "C" int b200_seq_diff_combine(const float* in, void* out, int out_dt, int64_t T, int H, int dv, float lambda, float out_scale, float eps,
                                     void* stream) {
  if (T == 0) return B200_OK;
  B200_SEQ_DISPATCH(out_dt, E, B200_LAUNCH((diff_combine_kernel<E>), dim3((unsigned)T), dim3(256), 0, (cudaStream_t)stream, in, (E*)out, H, dv, lambda,
                                           out_scale, eps));
  b200_count_launches(1);
  return B200_OK;
}
