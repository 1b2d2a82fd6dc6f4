// Latent attention over a paged latent cache.
//
// A token caches ONE row of D = R + r elements per layer: its normalised latent c (R) and its rotated shared key part (r).
// Attention runs in the absorbed form: a head's query is carried into latent space once (q~ = Wuk_h^T q_plain, done by the
// per-head product in seq_linear.cu), so that score(i, j) = (q~_i . c_j + qrot_i . krot_j) * scale and the head's output is
// Wuv_h (sum_j p_ij c_j): every head reads the same cache row, nothing per head is ever stored.
//
//   latent_prepare_kernel : RMS-norms the latent slice of the down-projection, rotates the shared key part, writes both into the
//                           token's cache slot; rotates each head's query part into the absorbed-query buffer.
//   latent_attn_kernel    : one block per (query token, group of heads), one warp per head; streams the visible window
//                           [p - window + 1, p] of the sequence's pages in tiles of 32 keys through shared memory, fp32 online
//                           soft-max.  Serves prompts, portions of prompts that follow cached tokens and single decoded tokens
//                           alike: a query's keys are always read back from the cache, whatever step wrote them.
//
// Rotation: interleaved pairs (2i, 2i+1) of the first `rot_dims` elements, angle tables [positions, rot_dims/2] (fp32, made
// by the host with any frequency scaling and amplitude factor folded in); elements past rot_dims pass unchanged.
#include "seq_common.cuh"

#include <cstdlib>

namespace b200 {
namespace seq {

constexpr int kPrepThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kPrepThreads) latent_prepare_kernel(
    const float* __restrict__ down, int64_t ld_down, int col_c, int col_kr,  // down-projection row: latent at col_c, key part at col_kr
    const float* __restrict__ q, int64_t ld_q, int q_head_stride, int q_rot_off,  // per head: rotated part at h*stride + off
    const T* __restrict__ cnorm_w, const float* __restrict__ cos_t, const float* __restrict__ sin_t, const int64_t* __restrict__ position_ids,
    const int64_t* __restrict__ slot_mapping, T* __restrict__ cache, float* __restrict__ q_abs, int H, int R, int r, int rot_dims, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  const int D = R + r, half = rot_dims / 2;
  const int64_t pos = position_ids[t];
  const int64_t slot = slot_mapping[t];
  const float* crow = down + t * ld_down + col_c;
  float s = 0.f;
  for (int i = threadIdx.x; i < R; i += kPrepThreads) s += crow[i] * crow[i];
  const float rstd = 1.f / sqrtf(block_sum(s, red) / R + eps);
  const float* cs = cos_t + pos * half;
  const float* sn = sin_t + pos * half;
  if (slot >= 0) {
    T* dst = cache + slot * D;
    for (int i = threadIdx.x; i < R; i += kPrepThreads) stf(dst + i, crow[i] * rstd * ldf(cnorm_w + i));
    const float* kr = down + t * ld_down + col_kr;
    for (int i = threadIdx.x; i < r; i += kPrepThreads) {
      float v;
      if (i < rot_dims) {
        const int p = i >> 1;
        const float a = kr[2 * p], b = kr[2 * p + 1];
        v = (i & 1) ? b * cs[p] + a * sn[p] : a * cs[p] - b * sn[p];
      } else {
        v = kr[i];
      }
      stf(dst + R + i, v);
    }
  }
  for (int idx = threadIdx.x; idx < H * r; idx += kPrepThreads) {
    const int h = idx / r, i = idx % r;
    const float* qr = q + t * ld_q + (int64_t)h * q_head_stride + q_rot_off;
    float v;
    if (i < rot_dims) {
      const int p = i >> 1;
      const float a = qr[2 * p], b = qr[2 * p + 1];
      v = (i & 1) ? b * cs[p] + a * sn[p] : a * cs[p] - b * sn[p];
    } else {
      v = qr[i];
    }
    q_abs[(t * H + h) * D + R + i] = v;
  }
}

constexpr int kHeadsPerBlock = 8, kKeyTile = 32;

template <typename T, int NR>
__global__ void __launch_bounds__(kHeadsPerBlock * 32) latent_attn_kernel(
    const float* __restrict__ q_abs, const T* __restrict__ cache, const int32_t* __restrict__ block_table, int64_t bt_stride,
    const int32_t* __restrict__ seq_of_token, const int64_t* __restrict__ position_ids, float* __restrict__ out, int H, int R, int D, int window,
    float scale, int page) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  float* qs = sm;                        // [kHeadsPerBlock][D]
  float* ks = sm + kHeadsPerBlock * D;   // [kKeyTile][D + 1]
  const int64_t t = blockIdx.x;
  const int h0 = blockIdx.y * kHeadsPerBlock;
  const int w = warp_id(), lane = lane_id();
  const int h = h0 + w;
  const int b = seq_of_token[t];
  const int p = (int)position_ids[t];
  const int j_lo = max(0, p - window + 1);
  const int nthreads = kHeadsPerBlock * 32;
  for (int idx = threadIdx.x; idx < kHeadsPerBlock * D; idx += nthreads) {
    const int hh = h0 + idx / D;
    qs[idx] = hh < H ? q_abs[(t * H + hh) * D + idx % D] : 0.f;
  }
  float m = -INFINITY, l = 0.f;
  float acc[NR];
#pragma unroll
  for (int i = 0; i < NR; ++i) acc[i] = 0.f;
  const int32_t* table = block_table + (int64_t)b * bt_stride;
  for (int j0 = j_lo; j0 <= p; j0 += kKeyTile) {
    __syncthreads();  // the previous tile is consumed (and qs is written, first time round)
    const int nk = min(kKeyTile, p - j0 + 1);
    for (int idx = threadIdx.x; idx < nk * D; idx += nthreads) {
      const int jj = idx / D, dd = idx % D;
      const int j = j0 + jj;
      const int64_t row = (int64_t)table[j / page] * page + j % page;
      ks[jj * (D + 1) + dd] = ldf(cache + row * D + dd);
    }
    __syncthreads();
    if (h < H) {
      float s = -INFINITY;
      if (lane < nk) {
        float a = 0.f;
        const float* kq = ks + lane * (D + 1);
        const float* qq = qs + w * D;
        for (int d = 0; d < D; ++d) a = fmaf(qq[d], kq[d], a);
        s = a * scale;
      }
      const float m_new = fmaxf(m, warp_max(s));
      const float pr = lane < nk ? expf(s - m_new) : 0.f;
      const float corr = expf(m - m_new);  // m = -inf on the first tile: 0
      l = l * corr + warp_sum(pr);
      m = m_new;
#pragma unroll
      for (int i = 0; i < NR; ++i) acc[i] *= corr;
      for (int jj = 0; jj < nk; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, pr, jj);
        const float* kr = ks + jj * (D + 1);
#pragma unroll
        for (int i = 0; i < NR; ++i) {
          const int d = lane + 32 * i;
          if (d < R) acc[i] = fmaf(pj, kr[d], acc[i]);
        }
      }
    }
  }
  if (h < H) {
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < NR; ++i) {
      const int d = lane + 32 * i;
      if (d < R) out[(t * H + h) * R + d] = acc[i] * inv;
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------------
// Tensor-core form for bfloat16 caches.  One block per (query token, 16 heads): the 16 heads are the M rows of m16n8k16 MMAs, so
// one pass over the token's window serves them all - the cache row of a key is the B operand of S = Q K^T (all D columns) and,
// read transposed, of O += P V (its first R columns).  Key tiles of 64 rows come in with 16-byte cp.async; each of the four warps
// scores 16 keys of the tile, the row maxima and sums meet in shared memory (fp32 online soft-max, every warp keeps the same
// running max and sum), P goes to shared memory as bfloat16, and each warp accumulates a quarter of the R output columns in
// registers.  Needs D % 16 == 0, R % 64 == 0, R <= 512; other shapes and float32 caches take latent_attn_kernel above.
// ------------------------------------------------------------------------------------------------------------------------
constexpr int kMmaKeys = 64, kMmaThreads = 128, kMmaPad = 8;
static_assert(kMmaThreads == 2 * kMmaKeys, "the tile loader pairs two threads with a key row");

template <int NTW>  // n-tiles (8 output columns each) per warp: R = 32 * NTW
__global__ void __launch_bounds__(kMmaThreads) latent_attn_mma_kernel(
    const float* __restrict__ q_abs, const __nv_bfloat16* __restrict__ cache, const int32_t* __restrict__ block_table, int64_t bt_stride,
    const int32_t* __restrict__ seq_of_token, const int64_t* __restrict__ position_ids, float* __restrict__ out, int H, int R, int D, int window,
    float scale, int page, float* __restrict__ partial) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int DP = D + kMmaPad;                // padded row (elements): rows 16 bytes apart modulo 128 -> conflict-free ldmatrix
  constexpr int PP = kMmaKeys + kMmaPad;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [16][DP]
  __nv_bfloat16* Ks = Qs + 16 * DP;                                  // [64][DP]
  __nv_bfloat16* Ps = Ks + kMmaKeys * DP;                            // [16][PP]
  float* red_max = reinterpret_cast<float*>(Ps + 16 * PP);           // [4][16]
  float* red_sum = red_max + 64;                                     // [4][16]
  const int64_t t = blockIdx.x;
  const int h0 = blockIdx.y * 16;
  const int w = warp_id(), lane = lane_id();
  const int b = seq_of_token[t];
  const int p = (int)position_ids[t];
  const int j_first = max(0, p - window + 1);
  // gridDim.z > 1: the token's key tiles are dealt out in contiguous runs to gridDim.z blocks, whose (max, sum, unnormalised O) per
  // head are merged by latent_attn_merge_kernel; a block whose run is empty records an empty partial
  const int n_tiles = (p - j_first + kMmaKeys) / kMmaKeys;
  const int per_split = (n_tiles + gridDim.z - 1) / gridDim.z;
  const int j_lo = j_first + (int)blockIdx.z * per_split * kMmaKeys;
  const int j_hi = min(p, j_lo + per_split * kMmaKeys - 1);
  const int32_t* table = block_table + (int64_t)b * bt_stride;
  for (int idx = threadIdx.x; idx < 16 * D; idx += kMmaThreads) {
    const int row = idx / D, d = idx % D;
    const float v = (h0 + row < H) ? q_abs[(t * H + h0 + row) * D + d] * scale : 0.f;
    Qs[row * DP + d] = __float2bfloat16_rn(v);
  }
  const int r0 = lane >> 2, cq = (lane & 3) * 2;   // accumulator rows r0, r0 + 8; columns cq, cq + 1 of an 8-wide tile
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[NTW][4];
#pragma unroll
  for (int i = 0; i < NTW; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const int chunks = D / 8;  // 16-byte pieces of a cache row
  const uint32_t qs_addr = smem_u32(Qs), ks_addr = smem_u32(Ks), ps_addr = smem_u32(Ps);
  for (int j0 = j_lo; j0 <= j_hi; j0 += kMmaKeys) {
    __syncthreads();  // everyone is done with the previous tile (and Qs is written, first time round)
    {
      // two threads per key row: one block-table lookup per thread and tile, then the row's 16-byte pieces alternate between them
      const int row = threadIdx.x >> 1, j = j0 + row;
      __nv_bfloat16* dst = Ks + row * DP;
      if (j <= p) {
        const __nv_bfloat16* src = cache + ((int64_t)table[j / page] * page + j % page) * D;
        for (int ch = threadIdx.x & 1; ch < chunks; ch += 2) cp_async_16(dst + ch * 8, src + ch * 8, true);
      } else {
        for (int ch = threadIdx.x & 1; ch < chunks; ch += 2)
          *reinterpret_cast<uint4*>(dst + ch * 8) = make_uint4(0u, 0u, 0u, 0u);  // finite: these rows meet p = 0
      }
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    // ---- S = Q K^T for this warp's 16 keys
    float s[2][4] = {};
    {
      const int m = lane >> 3, rr = lane & 7;
      const uint32_t a_lane = qs_addr + (uint32_t)((((m & 1) * 8 + rr) * DP + (m >> 1) * 8) * 2);
      const uint32_t b_lane = ks_addr + (uint32_t)(((w * 16 + (m >> 1) * 8 + rr) * DP + (m & 1) * 8) * 2);
      for (int kk = 0; kk < D; kk += 16) {
        uint32_t a[4], bb[4];
        ldmatrix_x4(a[0], a[1], a[2], a[3], a_lane + kk * 2);
        ldmatrix_x4(bb[0], bb[1], bb[2], bb[3], b_lane + kk * 2);
        mma_m16n8k16_bf16f32(s[0], a, bb[0], bb[1]);
        mma_m16n8k16_bf16f32(s[1], a, bb[2], bb[3]);
      }
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j0 + w * 16 + nt * 8 + cq + (e & 1);
        if (j > p) s[nt][e] = -INFINITY;
        mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
      }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
    }
    if ((lane & 3) == 0) {
      red_max[w * 16 + r0] = mx[0];
      red_max[w * 16 + r0 + 8] = mx[1];
    }
    __syncthreads();
    float m_new[2], corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = r0 + i * 8;
      const float tm = fmaxf(fmaxf(red_max[row], red_max[16 + row]), fmaxf(red_max[32 + row], red_max[48 + row]));
      m_new[i] = fmaxf(m_run[i], tm);  // finite: key j0 is visible to every row
      corr[i] = expf(m_run[i] - m_new[i]);
      m_run[i] = m_new[i];
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const float p0 = expf(s[nt][0] - m_new[0]), p1 = expf(s[nt][1] - m_new[0]);
      const float p2 = expf(s[nt][2] - m_new[1]), p3 = expf(s[nt][3] - m_new[1]);
      const __nv_bfloat162 lo = __floats2bfloat162_rn(p0, p1), hi = __floats2bfloat162_rn(p2, p3);
      // the sums use the rounded probabilities: numerator and denominator see the same weights
      sum[0] += __low2float(lo) + __high2float(lo);
      sum[1] += __low2float(hi) + __high2float(hi);
      const int col = w * 16 + nt * 8 + cq;
      *reinterpret_cast<__nv_bfloat162*>(Ps + r0 * PP + col) = lo;
      *reinterpret_cast<__nv_bfloat162*>(Ps + (r0 + 8) * PP + col) = hi;
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
      sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
    }
    if ((lane & 3) == 0) {
      red_sum[w * 16 + r0] = sum[0];
      red_sum[w * 16 + r0 + 8] = sum[1];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = r0 + i * 8;
      l_run[i] = l_run[i] * corr[i] + ((red_sum[row] + red_sum[16 + row]) + (red_sum[32 + row] + red_sum[48 + row]));
    }
#pragma unroll
    for (int i = 0; i < NTW; ++i) {
      o[i][0] *= corr[0];
      o[i][1] *= corr[0];
      o[i][2] *= corr[1];
      o[i][3] *= corr[1];
    }
    // ---- O += P V over this warp's NTW * 8 output columns
    {
      const int m = lane >> 3, rr = lane & 7;
      const uint32_t a_lane = ps_addr + (uint32_t)((((m & 1) * 8 + rr) * PP + (m >> 1) * 8) * 2);
      const uint32_t v_lane = ks_addr + (uint32_t)((((m & 1) * 8 + rr) * DP + w * NTW * 8 + (m >> 1) * 8) * 2);
#pragma unroll
      for (int ks = 0; ks < kMmaKeys / 16; ++ks) {
        uint32_t a[4];
        ldmatrix_x4(a[0], a[1], a[2], a[3], a_lane + ks * 32);
#pragma unroll
        for (int nt = 0; nt < NTW; nt += 2) {
          uint32_t bb[4];
          ldmatrix_x4_trans(bb[0], bb[1], bb[2], bb[3], v_lane + (uint32_t)((ks * 16 * DP + nt * 8) * 2));
          mma_m16n8k16_bf16f32(o[nt], a, bb[0], bb[1]);
          mma_m16n8k16_bf16f32(o[nt + 1], a, bb[2], bb[3]);
        }
      }
    }
  }
  if (gridDim.z > 1) {
    // partial [token][head group][split][16 rows][R + 2]: unnormalised O, then the running max and sum
    float* base = partial + ((((int64_t)t * gridDim.y + blockIdx.y) * gridDim.z + blockIdx.z) * 16) * (R + 2);
#pragma unroll
    for (int nt = 0; nt < NTW; ++nt) {
      const int col = (w * NTW + nt) * 8 + cq;
      base[r0 * (R + 2) + col] = o[nt][0];
      base[r0 * (R + 2) + col + 1] = o[nt][1];
      base[(r0 + 8) * (R + 2) + col] = o[nt][2];
      base[(r0 + 8) * (R + 2) + col + 1] = o[nt][3];
    }
    if (w == 0 && (lane & 3) == 0) {
      base[r0 * (R + 2) + R] = m_run[0];
      base[r0 * (R + 2) + R + 1] = l_run[0];
      base[(r0 + 8) * (R + 2) + R] = m_run[1];
      base[(r0 + 8) * (R + 2) + R + 1] = l_run[1];
    }
    return;
  }
  const float inv0 = 1.f / l_run[0], inv1 = 1.f / l_run[1];
#pragma unroll
  for (int nt = 0; nt < NTW; ++nt) {
    const int col = (w * NTW + nt) * 8 + cq;
    if (h0 + r0 < H) {
      float* dst = out + (t * H + h0 + r0) * R + col;
      dst[0] = o[nt][0] * inv0;
      dst[1] = o[nt][1] * inv0;
    }
    if (h0 + r0 + 8 < H) {
      float* dst = out + (t * H + h0 + r0 + 8) * R + col;
      dst[0] = o[nt][2] * inv1;
      dst[1] = o[nt][3] * inv1;
    }
  }
}

// out[t, h] = sum_z e^(m_z - M) O_z / sum_z e^(m_z - M) l_z over the splits of latent_attn_mma_kernel; one warp per (token, head)
__global__ void latent_attn_merge_kernel(const float* __restrict__ partial, float* __restrict__ out, int64_t Tq, int H, int R, int groups, int nsplit) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t wid = (int64_t)blockIdx.x * (blockDim.x / 32) + warp_id();
  if (wid >= Tq * H) return;
  const int64_t t = wid / H;
  const int h = (int)(wid % H), g = h / 16, row = h % 16, lane = lane_id();
  const float* base = partial + (((t * groups + g) * nsplit) * 16 + row) * (R + 2);
  const int64_t zs = (int64_t)16 * (R + 2);
  constexpr int kMaxSplit = 8;
  float M = -INFINITY, wz[kMaxSplit];
#pragma unroll
  for (int z = 0; z < kMaxSplit; ++z) {
    wz[z] = z < nsplit ? base[z * zs + R] : -INFINITY;
    M = fmaxf(M, wz[z]);
  }
  float den = 0.f;
#pragma unroll
  for (int z = 0; z < kMaxSplit; ++z) {
    wz[z] = wz[z] > -INFINITY ? expf(wz[z] - M) : 0.f;  // an empty run carries no weight
    if (z < nsplit) den += wz[z] * base[z * zs + R + 1];
  }
  const float inv = 1.f / den;
  for (int c = lane; c < R; c += 32) {
    float acc = 0.f;
#pragma unroll
    for (int z = 0; z < kMaxSplit; ++z)
      if (z < nsplit) acc = fmaf(wz[z], base[z * zs + c], acc);
    out[(t * H + h) * R + c] = acc * inv;
  }
}

}  // namespace seq
}  // namespace b200

using namespace b200::seq;

extern "C" int b200_seq_latent_prepare(const float* down, int64_t ld_down, int col_c, int col_kr, const float* q, int64_t ld_q, int q_head_stride,
                                       int q_rot_off, const void* cnorm_w, const float* cos_t, const float* sin_t, const int64_t* position_ids,
                                       const int64_t* slot_mapping, void* cache, int dt, float* q_abs, int64_t T, int H, int R, int r, int rot_dims,
                                       float eps, void* stream) {
  if (T == 0) return B200_OK;
  if (rot_dims % 2 != 0 || rot_dims > r || rot_dims < 0) { b200_set_last_error("seq_latent_prepare: rot_dims must be even and <= r"); return B200_ERR_ARG; }
  B200_SEQ_DISPATCH(dt, E, B200_LAUNCH((latent_prepare_kernel<E>), dim3((unsigned)T), dim3(kPrepThreads), 0, (cudaStream_t)stream, down, ld_down, col_c,
                                       col_kr, q, ld_q, q_head_stride, q_rot_off, (const E*)cnorm_w, cos_t, sin_t, position_ids, slot_mapping,
                                       (E*)cache, q_abs, H, R, r, rot_dims, eps));
  b200_count_launches(1);
  return B200_OK;
}

template <typename T, int NR>
static int launch_latent_attn(const float* q_abs, const void* cache, const int32_t* block_table, int64_t bt_stride, const int32_t* seq_of_token,
                              const int64_t* position_ids, float* out, int64_t Tq, int H, int R, int D, int window, float scale, int page,
                              cudaStream_t st) {
  const size_t smem = ((size_t)kHeadsPerBlock * D + (size_t)kKeyTile * (D + 1)) * 4;
  if (smem > 200 * 1024) { b200_set_last_error("seq_latent_attn: cache row too wide"); return B200_ERR_ARG; }
  static bool cfg = false;
  if (!cfg) { cudaFuncSetAttribute(latent_attn_kernel<T, NR>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); cfg = true; }
  dim3 grid((unsigned)Tq, (unsigned)((H + kHeadsPerBlock - 1) / kHeadsPerBlock));
  B200_LAUNCH((latent_attn_kernel<T, NR>), grid, dim3(kHeadsPerBlock * 32), smem, st, q_abs, (const T*)cache, block_table, bt_stride, seq_of_token,
              position_ids, out, H, R, D, window, scale, page);
  b200_count_launches(1);
  return B200_OK;
}

// q_abs [Tq, H, D] fp32; cache [blocks, page, D] of type dt; out [Tq, H, R] fp32.  window <= 0: every earlier token is visible.
// Blocks the tensor-core kernel should split every token's keys over (1 = no split), and the fp32 workspace that needs: few tokens
// (decoding) leave most SMs idle with one block per (token, 16 heads).  0 when the shape takes the plain kernel.
extern "C" int b200_seq_latent_attn_splits(int dt, int64_t Tq, int H, int R, int r, int64_t* workspace_floats) {
  const int D = R + r;
  if (workspace_floats) *workspace_floats = 0;
  if (!(dt == B200_DT_BF16 && D % 16 == 0 && R % 64 == 0 && R <= 512)) return 0;
  const int64_t blocks = Tq * ((H + 15) / 16);
  int64_t n = (2 * 148) / (blocks > 0 ? blocks : 1);
  n = n < 1 ? 1 : (n > 8 ? 8 : n);
  if (n > 1 && workspace_floats) *workspace_floats = blocks * n * 16 * (R + 2);
  return (int)n;
}

// `partial` / nsplit: from b200_seq_latent_attn_splits (NULL / <= 1: no split).
extern "C" int b200_seq_latent_attn(const float* q_abs, const void* cache, int dt, const int32_t* block_table, int64_t bt_stride,
                                    const int32_t* seq_of_token, const int64_t* position_ids, float* out, int64_t Tq, int H, int R, int r,
                                    int window, float scale, int page, float* partial, int nsplit, void* stream) {
  if (Tq == 0) return B200_OK;
  const int D = R + r;
  if (window <= 0) window = 0x3fffffff;
  const int nr = (R + 31) / 32;
  cudaStream_t st = (cudaStream_t)stream;
  static const bool use_mma = []() { const char* e = getenv("B200_SEQ_ATTN_MMA"); return !(e && e[0] == '0'); }();
  if (use_mma && dt == B200_DT_BF16 && D % 16 == 0 && R % 64 == 0 && R <= 512 && (reinterpret_cast<uintptr_t>(cache) & 15) == 0) {
    const int ntw = R / 32;
    const size_t smem = ((size_t)(16 + kMmaKeys) * (D + kMmaPad) + 16 * (kMmaKeys + kMmaPad)) * 2 + 128 * 4;
    if (!partial || nsplit < 1) nsplit = 1;
    dim3 grid((unsigned)Tq, (unsigned)((H + 15) / 16), (unsigned)nsplit);
#define LAM(N)                                                                                                                        \
  do {                                                                                                                                \
    static bool cfg = false;                                                                                                          \
    if (!cfg) { cudaFuncSetAttribute(latent_attn_mma_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); cfg = true; } \
    B200_LAUNCH((latent_attn_mma_kernel<N>), grid, dim3(kMmaThreads), smem, st, q_abs, (const __nv_bfloat16*)cache, block_table, bt_stride, \
                seq_of_token, position_ids, out, H, R, D, window, scale, page, partial);                                              \
    if (nsplit > 1)                                                                                                                   \
      B200_LAUNCH(latent_attn_merge_kernel, dim3((unsigned)((Tq * H + 3) / 4)), dim3(128), 0, st, (const float*)partial, out, Tq, H, R, \
                  (int)grid.y, nsplit);                                                                                              \
    b200_count_launches(nsplit > 1 ? 2 : 1);                                                                                          \
    return B200_OK;                                                                                                                   \
  } while (0)
    switch (ntw) {
      case 2: LAM(2);
      case 4: LAM(4);
      case 6: LAM(6);
      case 8: LAM(8);
      case 10: LAM(10);
      case 12: LAM(12);
      case 14: LAM(14);
      case 16: LAM(16);
      default: break;
    }
#undef LAM
  }
#define LA(NR)                                                                                                                         \
  B200_SEQ_DISPATCH(dt, E, return (launch_latent_attn<E, NR>(q_abs, cache, block_table, bt_stride, seq_of_token, position_ids, out, Tq, H, R, D, \
                                                            window, scale, page, st)))
  if (nr <= 4) LA(4);
  else if (nr <= 8) LA(8);
  else if (nr <= 16) LA(16);
  else if (nr <= 32) LA(32);
#undef LA
  b200_set_last_error("seq_latent_attn: latent wider than 1024");
  return B200_ERR_UNSUPPORTED;
}
