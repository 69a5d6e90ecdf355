// tcgen05 / TMEM / TMA kernels: TF32 GEMM with FP32 accumulation for Linear layers, and
// implicit-GEMM convolution forward and (stride-1) data gradient over channels-last tensors.
//
// One persistent CTA per SM, 192 threads in three roles:
//   warp 0     TMA producer: one lane fills a ring of shared-memory stages (A tile 128 x 32,
//              B tile BN x 32 fp32, 128-byte swizzle).  The convolution's A operand is never
//              materialised: an im2col-mode tensor map gathers 128 output pixels x 32 channels
//              of one filter tap per load, with zero fill for the padding halo.
//   warp 1     MMA issuer: one lane issues tcgen05.mma kind::tf32 (128 x BN x 8 per instruction),
//              accumulating in TMEM; tcgen05.commit releases stages and publishes finished tiles.
//   warps 2-5  epilogue: tcgen05.ld the accumulator (each warp owns a 32-lane TMEM quarter),
//              add bias / apply ReLU, store rows to global memory.
// Two TMEM accumulator buffers let the epilogue of tile i overlap the main loop of tile i+1.
// All waits are bounded (tc_common.cuh); a kernel that gives up sets g_tc_status and exits.
#include "tc_common.cuh"
#include "kernels.h"
#include <cudaTypedefs.h>

namespace tc {

static PFN_cuTensorMapEncodeTiled_v12000 g_encode_tiled = nullptr;
static PFN_cuTensorMapEncodeIm2col_v12000 g_encode_im2col = nullptr;

// Element type recorded in the tensor maps.  TFLOAT32 makes the copy engine round every fp32
// value to TF32 on its way into shared memory (measured: max relative error of a K=1024 GEMM
// 2.7e-4, against 7.4e-4 when the raw fp32 bits are handed to the MMA, which then simply drops
// the low 13 mantissa bits).  MTB_TMA_FLOAT32=1 selects the unrounded variant for comparison.
static CUtensorMapDataType tma_dtype() {
  static int mode = -1;
  if (mode < 0) mode = getenv("MTB_TMA_FLOAT32") ? 1 : 0;
  return mode ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_TFLOAT32;
}

static int load_driver_entry_points() {
  if (g_encode_tiled && g_encode_im2col) return MTB_OK;
  cudaDriverEntryPointQueryResult q;
  void* fn = nullptr;
  MTB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
  if (q != cudaDriverEntryPointSuccess || !fn) return mtb_fail(MTB_ERR_CUDA, "cuTensorMapEncodeTiled is not available in this driver");
  g_encode_tiled = (PFN_cuTensorMapEncodeTiled_v12000)fn;
  fn = nullptr;
  MTB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &q));
  if (q != cudaDriverEntryPointSuccess || !fn) return mtb_fail(MTB_ERR_CUDA, "cuTensorMapEncodeIm2col is not available in this driver");
  g_encode_im2col = (PFN_cuTensorMapEncodeIm2col_v12000)fn;
  return MTB_OK;
}

int encode_tiled_2d(CUtensorMap* map, const float* base, long long rows, long long cols, long long pitch_elems, int box_cols, int box_rows,
                    bool mn_major) {
  int rc = load_driver_entry_points();
  if (rc) return rc;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)pitch_elems * 4};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode_tiled(map, tma_dtype(), 2, const_cast<float*>(base), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return mtb_fail(MTB_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) rows=%lld cols=%lld pitch=%lld box=%dx%d", (int)r, rows, cols, pitch_elems, box_cols, box_rows);
  return MTB_OK;
}

int encode_rows_4d(CUtensorMap* map, const float* base, int n, int h, int w, int c, int channels, int box_w, bool mn_major) {
  int rc = load_driver_entry_points();
  if (rc) return rc;
  cuuint64_t dims[4] = {(cuuint64_t)c, (cuuint64_t)w, (cuuint64_t)h, (cuuint64_t)n};
  cuuint64_t strides[3] = {(cuuint64_t)c * 4, (cuuint64_t)w * c * 4, (cuuint64_t)h * w * c * 4};
  cuuint32_t box[4] = {(cuuint32_t)channels, (cuuint32_t)box_w, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = g_encode_tiled(map, tma_dtype(), 4, const_cast<float*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return mtb_fail(MTB_ERR_CUDA, "cuTensorMapEncodeTiled (rows) failed (%d) n=%d h=%d w=%d c=%d box_w=%d", (int)r, n, h, w, c, box_w);
  return MTB_OK;
}

int encode_im2col_4d(CUtensorMap* map, const float* base, int n, int h, int w, int c, int lower_w, int lower_h, int upper_w, int upper_h,
                     int stride_w, int stride_h, int channels, int pixels, bool mn_major) {
  int rc = load_driver_entry_points();
  if (rc) return rc;
  cuuint64_t dims[4] = {(cuuint64_t)c, (cuuint64_t)w, (cuuint64_t)h, (cuuint64_t)n};
  cuuint64_t strides[3] = {(cuuint64_t)c * 4, (cuuint64_t)w * c * 4, (cuuint64_t)h * w * c * 4};
  int lower[2] = {lower_w, lower_h};
  int upper[2] = {upper_w, upper_h};
  cuuint32_t estr[4] = {1, (cuuint32_t)stride_w, (cuuint32_t)stride_h, 1};
  CUresult r = g_encode_im2col(map, tma_dtype(), 4, const_cast<float*>(base), dims, strides, lower, upper,
                               (cuuint32_t)channels, (cuuint32_t)pixels, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return mtb_fail(MTB_ERR_CUDA, "cuTensorMapEncodeIm2col failed (%d) n=%d h=%d w=%d c=%d lower=(%d,%d) upper=(%d,%d) stride=(%d,%d)", (int)r, n,
                    h, w, c, lower_w, lower_h, upper_w, upper_h, stride_w, stride_h);
  return MTB_OK;
}

}  // namespace tc

namespace {
using namespace tc;

enum { A_KMAJOR = 0, A_MNMAJOR = 1, A_IM2COL = 2 };
enum { B_KMAJOR = 0, B_MNMAJOR = 1 };

struct GemmParams {
  int M, N;
  int num_kb;  // reduction blocks of 32
  int m_tiles, n_tiles;
  float* out;
  long long ldo;
  const float* bias;
  // optional: out += result instead of out = result (the rows of `out` already hold a value this launch adds
  // to; a thread reads the very elements it then writes, so accumulating in place is safe)
  int accumulate;
  int relu;
  // geometry of the im2col'ed tensor (A operand of a convolution)
  int OW, OH, SW, SH, PW, PH, KW, KH, cchunks;
  // B operand addressed per filter tap (data gradient: weights read in place).  When set, the
  // k-block (tap, cc) reads B at inner coordinate b_tap_x[tap] + n0 (+32j), outer cc*32.
  int b_per_tap;
  int b_tap_x[64];
  // Output rows are pixels of a strided sub-grid of an [N, o_H, o_W, ldo] tensor: row
  // (n, i, j) of an o_Hc x o_Wc grid lands on pixel (o_h0 + o_sh*i, o_w0 + o_sw*j).
  int o_strided, o_Hc, o_Wc, o_H, o_W, o_h0, o_w0, o_sh, o_sw;
  // STATS kernels only: partial rows [(blockIdx.x / n_tiles) * 4 + epilogue warp][3][N] of per-column
  // (count, mean, M2) over the output rows this CTA produced (the grid is a multiple of n_tiles, so a
  // CTA always works on the same column tile)
  float* stats;
  // Split reduction (splits > 1): unit u = tile * splits + split works on reduction blocks
  // [split * kb_per_split, ...); every unit writes its raw accumulator to partial[u] and draws a ticket for
  // its tile; the unit that draws the last ticket adds the partials in split order and finishes the tile.
  int splits, kb_per_split;
  float* partial;
};

// One ticket counter per output tile of a split launch; back to zero when the launch ends.  Launches that
// split must not overlap on one GPU (they share the counters), which holds for work on one stream.
constexpr int kMaxSplitTiles = 1024;
static __device__ unsigned int g_gemm_tickets[kMaxSplitTiles];

// A stage holds kKB reduction blocks of 32 (each one 128-byte swizzle span per operand row).  One
// producer/consumer hand-over costs the issuing thread 300-400 cycles that do not overlap with MMA
// work, and four MMAs of a narrow tile are only 192-256 cycles of work, so tiles up to 128 wide
// take two blocks (8 MMAs) per stage.
template <int BN>
struct Cfg {
  static constexpr int kKB = BN <= 128 ? 2 : 1;
  static constexpr int kStages = BN == 256 ? 4 : (BN == 128 ? 3 : 4);
  static constexpr uint32_t kABytes = 128 * 32 * 4;   // one reduction block of A
  static constexpr uint32_t kBBytes = BN * 32 * 4;    // one reduction block of B
  static constexpr uint32_t kStageBytes = kKB * (kABytes + kBBytes);  // [A blocks][B blocks]
  static constexpr uint32_t kSmemBytes = kStages * kStageBytes + 1024;  // + alignment slack
  static constexpr uint32_t kTmemCols = 2 * BN;
};

template <int BN, int AMODE, int BMODE, bool STATS>
__global__ void __launch_bounds__(192, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const GemmParams p) {
  using C = Cfg<BN>;
  constexpr int STAGES = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_full[8], bar_empty[8], bar_tfull[2], bar_tempty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ int split_last;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_tfull[b]), 1);
      mbar_init(smem_u32(&bar_tempty[b]), 4);  // one arrival per epilogue warp
    }
    abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  const int S = p.splits;
  const int tiles = p.m_tiles * p.n_tiles * S;  // work units: (tile, split) pairs, the splits of a tile adjacent
  volatile int* abort_ptr = &abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&mapA);
      prefetch_tensormap(&mapB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < tiles && ok; unit += gridDim.x) {
        const int tile = unit / S, split = unit - tile * S;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = kb0 + p.kb_per_split < p.num_kb ? kb0 + p.kb_per_split : p.num_kb;
        const int m0 = (tile / p.n_tiles) * 128, n0 = (tile % p.n_tiles) * BN;
        int pix_w = 0, pix_h = 0, pix_n = 0;
        if (AMODE == A_IM2COL) {
          int ow = m0 % p.OW, t = m0 / p.OW;
          pix_w = ow * p.SW - p.PW;
          pix_h = (t % p.OH) * p.SH - p.PH;
          pix_n = t / p.OH;
        }
        // reduction blocks in (tap, channel-block) order; plain GEMMs have a single "tap"
        int cc = kb0 % p.cchunks, kw = (kb0 / p.cchunks) % p.KW, kh = (kb0 / p.cchunks) / p.KW;
        for (int kb = kb0; kb < kb1 && ok; kb += C::kKB) {
          const int nblk = kb1 - kb < C::kKB ? kb1 - kb : C::kKB;  // the last stage may hold one block
          if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abort_ptr, 1)) { ok = false; break; }
          const uint32_t full = smem_u32(&bar_full[stage]);
          mbar_expect_tx(full, (uint32_t)nblk * (C::kABytes + C::kBBytes));
          const uint32_t st_base = smem_base + stage * C::kStageBytes;
          for (int h = 0; h < nblk; ++h) {
            const int kbh = kb + h;
            const int tap = kh * p.KW + kw;
            const uint32_t a_dst = st_base + h * C::kABytes, b_dst = st_base + C::kKB * C::kABytes + h * C::kBBytes;
            if (AMODE == A_KMAJOR) {
              tma_load_2d(a_dst, &mapA, full, kbh * 32, m0);
            } else if (AMODE == A_MNMAJOR) {
#pragma unroll
              for (int j = 0; j < 4; ++j) tma_load_2d(a_dst + j * 4096, &mapA, full, m0 + 32 * j, kbh * 32);
            } else {
              tma_load_im2col_4d(a_dst, &mapA, full, cc * 32, pix_w, pix_h, pix_n, (uint16_t)kw, (uint16_t)kh);
            }
            if (BMODE == B_KMAJOR) {
              tma_load_2d(b_dst, &mapB, full, kbh * 32, n0);
            } else {
              int bx = n0, by = kbh * 32;
              if (p.b_per_tap) { bx = p.b_tap_x[tap] + n0; by = cc * 32; }
#pragma unroll
              for (int j = 0; j < BN / 32; ++j) tma_load_2d(b_dst + j * 4096, &mapB, full, bx + 32 * j, by);
            }
            if (++cc == p.cchunks) {
              cc = 0;
              if (++kw == p.KW) { kw = 0; ++kh; }
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // The whole warp runs the loop converged and one elected lane issues (warp-uniform control
    // flow keeps the descriptors in uniform registers: a lane-0 branch around the loop costs
    // about twice as many cycles per tcgen05.mma).
    constexpr uint32_t idesc = idesc_tf32(128, BN, AMODE == A_MNMAJOR ? 1 : 0, BMODE == B_MNMAJOR ? 1 : 0);
    constexpr uint32_t a_hi = AMODE == A_MNMAJOR ? desc_hi_mnmajor() : desc_hi_kmajor();
    constexpr uint32_t b_hi = BMODE == B_MNMAJOR ? desc_hi_mnmajor() : desc_hi_kmajor();
    constexpr uint32_t a_step = AMODE == A_MNMAJOR ? (1024u >> 4) : (32u >> 4);  // per 8 of K, in 16-byte units
    constexpr uint32_t b_step = BMODE == B_MNMAJOR ? (1024u >> 4) : (32u >> 4);
    const uint32_t a_lo0 = AMODE == A_MNMAJOR ? desc_lo_mnmajor(smem_base) : desc_lo_kmajor(smem_base);
    const uint32_t b_lo0 = BMODE == B_MNMAJOR ? desc_lo_mnmajor(smem_base + C::kKB * C::kABytes) : desc_lo_kmajor(smem_base + C::kKB * C::kABytes);
    int stage = 0;
    uint32_t phase = 0;
    int t = 0;
    bool ok = true;
    for (int unit = blockIdx.x; unit < tiles && ok; unit += gridDim.x, ++t) {
      const int split = unit % S;
      const int kb0 = split * p.kb_per_split;
      const int kb1 = kb0 + p.kb_per_split < p.num_kb ? kb0 + p.kb_per_split : p.num_kb;
      const int buf = t & 1;
      const uint32_t use = (uint32_t)(t >> 1);
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_tempty[buf]), (use & 1u) ^ 1u, abort_ptr, 2));
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + buf * BN;
      uint32_t acc = 0;
      for (int kb = kb0; kb < kb1; kb += C::kKB) {
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_full[stage]), phase, abort_ptr, 3));
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_lo = a_lo0 + stage * (C::kStageBytes >> 4), b_lo = b_lo0 + stage * (C::kStageBytes >> 4);
        const bool second = C::kKB == 2 && kb + 1 < kb1;
        if (elect_one()) {
          mma_tf32_words(d_tmem, a_lo, a_hi, b_lo, b_hi, idesc, acc);
          mma_tf32_words(d_tmem, a_lo + a_step, a_hi, b_lo + b_step, b_hi, idesc, 1u);
          mma_tf32_words(d_tmem, a_lo + 2 * a_step, a_hi, b_lo + 2 * b_step, b_hi, idesc, 1u);
          mma_tf32_words(d_tmem, a_lo + 3 * a_step, a_hi, b_lo + 3 * b_step, b_hi, idesc, 1u);
          if (second) {
            constexpr uint32_t a2 = C::kABytes >> 4, b2 = C::kBBytes >> 4;
            mma_tf32_words(d_tmem, a_lo + a2, a_hi, b_lo + b2, b_hi, idesc, 1u);
            mma_tf32_words(d_tmem, a_lo + a2 + a_step, a_hi, b_lo + b2 + b_step, b_hi, idesc, 1u);
            mma_tf32_words(d_tmem, a_lo + a2 + 2 * a_step, a_hi, b_lo + b2 + 2 * b_step, b_hi, idesc, 1u);
            mma_tf32_words(d_tmem, a_lo + a2 + 3 * a_step, a_hi, b_lo + b2 + 3 * b_step, b_hi, idesc, 1u);
          }
          mma_commit(smem_u32(&bar_empty[stage]));
        }
        __syncwarp();
        acc = 1u;
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
      if (ok && elect_one()) mma_commit(smem_u32(&bar_tfull[buf]));
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;
    int t = 0;
    const bool vec_ok = (p.ldo % 4 == 0) && (((reinterpret_cast<uintptr_t>(p.out) | reinterpret_cast<uintptr_t>(p.bias)) & 15u) == 0);
    const bool wide_ok = vec_ok && (p.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 31u) == 0);  // 32-byte stores
    // statistics variant: narrow tiles keep per-lane sums (cheap per tile), wide tiles merge per tile
    constexpr bool LANE_SUMS = STATS && BN == 64;
    WarpColStats<(STATS && !LANE_SUMS) ? BN / 32 : 1> stats;
    LaneColSums<LANE_SUMS ? BN / 32 : 1> sums;
    if constexpr (LANE_SUMS) sums.reset(); else stats.reset();
    for (int unit = blockIdx.x; unit < tiles; unit += gridDim.x, ++t) {
      const int tile = unit / S;
      const int m0 = (tile / p.n_tiles) * 128, n0 = (tile % p.n_tiles) * BN;
      const int buf = t & 1;
      const uint32_t use = (uint32_t)(t >> 1);
      // one lane polls (128 threads spinning on the barrier slow the other roles' barrier traffic down)
      bool ok = lane != 0 || mbar_wait(smem_u32(&bar_tfull[buf]), use & 1u, abort_ptr, 4);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      long long orow_index = row;
      if (p.o_strided && row < p.M) {
        const int j = row % p.o_Wc, t2 = row / p.o_Wc;
        const int i = t2 % p.o_Hc, nn = t2 / p.o_Hc;
        orow_index = ((long long)nn * p.o_H + p.o_h0 + p.o_sh * i) * p.o_W + p.o_w0 + p.o_sw * j;
      }
      float* orow = p.out + orow_index * p.ldo;
      const bool valid = row < p.M;
      const float cnt = STATS ? (float)__popc(__ballot_sync(0xffffffffu, valid)) : 0.f;
      // r: this lane's row of the finished accumulator, columns c0 .. c0+31 of the tile
      auto finish = [&](int c0, const uint32_t (&r)[32]) {
        const int col0 = n0 + c0;
        if constexpr (STATS) {
          // the forward convolution that feeds a BatchNorm layer: full column tiles (N % 32 == 0, checked on
          // the host), vector stores, and the per-channel statistics of what is stored
          if (col0 < p.N) {  // warp-uniform
            float o[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = __uint_as_float(r[j]) + (p.bias ? __ldg(p.bias + col0 + j) : 0.f);
            if (valid) {
#pragma unroll
              for (int j = 0; j < 32; j += 8)
                st_row8(orow + col0 + j, make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]), make_float4(o[j + 4], o[j + 5], o[j + 6], o[j + 7]), wide_ok);
            }
            if constexpr (LANE_SUMS) {
              if (valid) sums.add_chunk(c0 / 32, r);
            } else {
              if (cnt > 0.f) stats.add_chunk(c0 / 32, o, valid, cnt, lane);
            }
          }
        } else {
          if (valid && col0 < p.N) {
            if (vec_ok && col0 + 32 <= p.N) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                float4 v[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                  const int jj = j + 4 * h;
                  v[h] = make_float4(__uint_as_float(r[jj]), __uint_as_float(r[jj + 1]), __uint_as_float(r[jj + 2]), __uint_as_float(r[jj + 3]));
                  if (p.bias) {
                    const float4 b = *reinterpret_cast<const float4*>(p.bias + col0 + jj);
                    v[h].x += b.x; v[h].y += b.y; v[h].z += b.z; v[h].w += b.w;
                  }
                  if (p.accumulate) {
                    const float4 b = *reinterpret_cast<const float4*>(orow + col0 + jj);
                    v[h].x += b.x; v[h].y += b.y; v[h].z += b.z; v[h].w += b.w;
                  }
                  if (p.relu) { v[h].x = fmaxf(v[h].x, 0.f); v[h].y = fmaxf(v[h].y, 0.f); v[h].z = fmaxf(v[h].z, 0.f); v[h].w = fmaxf(v[h].w, 0.f); }
                }
                st_row8(orow + col0 + j, v[0], v[1], wide_ok);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (col0 + j < p.N) {
                  float v = __uint_as_float(r[j]);
                  if (p.bias) v += p.bias[col0 + j];
                  if (p.accumulate) v += orow[col0 + j];
                  if (p.relu) v = fmaxf(v, 0.f);
                  orow[col0 + j] = v;
                }
              }
            }
          }
        }
      };
      auto release_accumulator = [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[buf]));
      };
      auto count_rows = [&]() {
        if constexpr (LANE_SUMS) sums.cnt += valid ? 1.f : 0.f;
        else if constexpr (STATS) stats.n += cnt;
      };
      if (S == 1) {
        if constexpr (STATS) {
#pragma unroll
          for (int c0 = 0; c0 < BN; c0 += 32) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c0), r);
            tmem_ld_wait();
            finish(c0, r);
          }
        } else {
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 32) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c0), r);
            tmem_ld_wait();
            finish(c0, r);
          }
        }
        count_rows();
        release_accumulator();
        continue;
      }
      // Split reduction.  partial[unit][chunk][quarter][j][lane]: a warp stores 128 contiguous bytes per column.
      constexpr int kChunks = BN / 32;
      float* part = p.partial + (((long long)unit * kChunks) * 4 + quarter) * 1024 + lane;
#pragma unroll 1
      for (int c = 0; c < kChunks; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c * 32), r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) part[c * 4096 + j * 32] = __uint_as_float(r[j]);
      }
      release_accumulator();
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
      if (threadIdx.x == 64) {
        const unsigned int ticket = atomicAdd(&g_gemm_tickets[tile], 1u);
        split_last = (ticket == (unsigned int)S - 1u);
        if (split_last) g_gemm_tickets[tile] = 0u;  // every unit of the tile has drawn: ready for the next launch
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (!split_last) continue;
      __threadfence();
      const float* first = p.partial + (((long long)tile * S * kChunks) * 4 + quarter) * 1024 + lane;
      auto reduce_chunk = [&](int c, uint32_t (&r)[32]) {
        float acc[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = __ldcg(first + c * 4096 + j * 32);
        for (int sp = 1; sp < S; ++sp) {  // fixed order: split 0, 1, 2, ...
          const float* q = first + (long long)sp * kChunks * 4096 + c * 4096;
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[j] += __ldcg(q + j * 32);
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(acc[j]);
      };
      if constexpr (STATS) {
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
          uint32_t r[32];
          reduce_chunk(c, r);
          finish(c * 32, r);
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < kChunks; ++c) {
          uint32_t r[32];
          reduce_chunk(c, r);
          finish(c * 32, r);
        }
      }
      count_rows();
      if constexpr (STATS) {
        // which unit of a tile comes last differs from run to run, so the statistics of a split tile go to
        // a row chosen by the tile, not by the CTA: results stay bit-reproducible
        float* row = p.stats + ((long long)(tile / p.n_tiles) * 4 + quarter) * 3 * p.N;
        if constexpr (LANE_SUMS) { sums.store(row, p.N, n0, p.N, p.bias, lane); sums.reset(); }
        else { stats.store(row, p.N, n0, p.N, lane); stats.reset(); }
      }
    }
    if (STATS && S == 1) {
      float* row = p.stats + ((long long)(blockIdx.x / p.n_tiles) * 4 + quarter) * 3 * p.N;
      if constexpr (LANE_SUMS) sums.store(row, p.N, (blockIdx.x % p.n_tiles) * BN, p.N, p.bias, lane);
      else if constexpr (STATS) stats.store(row, p.N, (blockIdx.x % p.n_tiles) * BN, p.N, lane);
    }
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
    // give copies that are still in flight time to land before the CTA's shared memory is released
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int BN, int AMODE, int BMODE, bool STATS = false>
int launch_tc(const CUtensorMap& mapA, const CUtensorMap& mapB, const GemmParams& p, cudaStream_t st) {
  using C = Cfg<BN>;
  auto kernel = tc_gemm_kernel<BN, AMODE, BMODE, STATS>;
  static unsigned long long configured = 0;
  if (int rc = mtb_opt_in_smem((const void*)kernel, (int)C::kSmemBytes, &configured)) return rc;
  int tiles = p.m_tiles * p.n_tiles * p.splits;  // work units
  int grid = tiles < mtb_sm_count() ? tiles : mtb_sm_count();
  if (STATS && p.splits == 1) grid = grid / p.n_tiles * p.n_tiles;  // every CTA stays on one column tile (see GemmParams::stats)
  kernel<<<grid, 192, C::kSmemBytes, st>>>(mapA, mapB, p);
  MTB_LAUNCH_CHECK("tc_gemm_kernel");
  return MTB_OK;
}

// Partial-statistics rows the STATS variant writes for a problem of `tiles` tiles in `n_tiles` column tiles.
int stats_rows_for(int tiles, int n_tiles) {
  int grid = tiles < mtb_sm_count() ? tiles : mtb_sm_count();
  return grid / n_tiles * 4;
}

template <int AMODE, int BMODE>
int launch_tc_bn(int bn, const CUtensorMap& mapA, const CUtensorMap& mapB, const GemmParams& p, cudaStream_t st) {
  if (bn == 64) return launch_tc<64, AMODE, BMODE>(mapA, mapB, p, st);
  if (bn == 128) return launch_tc<128, AMODE, BMODE>(mapA, mapB, p, st);
  return launch_tc<256, AMODE, BMODE>(mapA, mapB, p, st);
}

int pick_bn(int n) { return n <= 64 ? 64 : (n <= 128 ? 128 : 256); }

// Tile width for a GEMM with `rows` output rows: the widest tile (best MMA efficiency) that still
// yields enough tiles to occupy most SMs; small problems (late layers at small batch) fall back
// to narrower tiles so that more CTAs take part.
int pick_bn_for(int n, long long rows) {
  const long long m_tiles = (rows + 127) / 128;
  const int want = mtb_sm_count() * 3 / 4;
  int bn = pick_bn(n);
  while (bn > 64 && m_tiles * ((n + bn - 1) / bn) < want) bn >>= 1;
  return bn;
}

// Tile width and reduction split for the im2col / GEMM kernel.  These kernels are bound by what one SM
// can pull from L2 into shared memory (about 89 GB/s: 47 B per cycle), then by the MMA rate, so a launch
// is priced as waves x reduction blocks per unit x the slower of (bytes of one block of A and B at that
// rate, four MMAs), plus, for a split reduction, the last unit's pass over the partials.  The cheapest
// (tile width, splits) wins; a split is only considered when all its units fit the GPU at once
// (tiles x splits <= SMs) and every unit keeps at least eight reduction blocks.
struct GemmPlan { int bn, splits, kb_per_split; };

GemmPlan plan_gemm(int n, long long rows, int num_kb, bool may_split, int force_bn = 0) {
  const int sms = mtb_sm_count();
  const long long m_tiles = (rows + 127) / 128;
  static const int kSplits[] = {1, 2, 3, 4, 6, 8};
  GemmPlan best{force_bn ? force_bn : pick_bn_for(n, rows), 1, num_kb};
  // Measured: the split only pays when even 64-wide tiles leave half the GPU idle (the 4x4 layers at 64
  // images: 41 -> 24 us for the data gradient of 512 -> 512); with more tiles than that the last unit's pass
  // over the partials costs more than the idle SMs did (256 -> 256 on 8x8 at 64 images: 20 -> 40 us).
  if (m_tiles * ((n + 63) / 64) > sms / 2 || num_kb < 64) may_split = false;  // short reductions gain nothing either
  if (!may_split || getenv("MTB_DISABLE_SPLITK")) return best;
  double best_ns = 1e30;
  for (int bn = force_bn ? force_bn : pick_bn(n); bn >= (force_bn ? force_bn : 64); bn >>= 1) {
    const long long tiles = m_tiles * ((n + bn - 1) / bn);
    for (int want : kSplits) {
      if (want > 1 && (tiles * want > sms || num_kb / want < 8 || tiles > kMaxSplitTiles)) continue;
      const int per = (num_kb + want - 1) / want;
      const int splits = (num_kb + per - 1) / per;
      const long long waves = (tiles * splits + sms - 1) / sms;
      const double load_ns = (16384.0 + bn * 128.0) / 89.0;
      const double mma_ns = 4.0 * (bn == 64 ? 48.0 : bn == 128 ? 64.0 : 128.0) / 1.9;
      double ns = (double)waves * per * (load_ns > mma_ns ? load_ns : mma_ns) + 2000.0;
      if (splits > 1) ns += splits * 128.0 * bn * 4.0 / 150.0 + 1500.0;
      if (ns < best_ns) { best_ns = ns; best = GemmPlan{bn, splits, per}; }
    }
  }
  return best;
}

long long split_partial_bytes(const GemmPlan& g, long long rows, int n) {
  if (g.splits <= 1) return 0;
  const long long tiles = ((rows + 127) / 128) * ((n + g.bn - 1) / g.bn);
  return tiles * g.splits * 128LL * g.bn * 4;
}

bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Activations smaller than this stay on the CUDA-core kernels: tiny tensors gain nothing from
// the tensor cores, and im2col tensor maps over very small tensors are avoided altogether.
constexpr long long kMinIm2colBytes = 128 * 1024;

}  // namespace

#include "tc_conv_rows.cuh"

// ------------------------------------------------------------------------------ host API

// Reads (and clears) the status word the tensor-core kernels set when a bounded wait ran out.
// Synchronises the device.
MTB_API int mtb_tc_status(int* status_out) {
  int h[8] = {0};
  MTB_CUDA(cudaDeviceSynchronize());
  MTB_CUDA(cudaMemcpyFromSymbol(h, g_tc_status, sizeof(h)));
  if (status_out) *status_out = h[0];
  if (h[0] != 0) {
    int z[8] = {0};
    MTB_CUDA(cudaMemcpyToSymbol(g_tc_status, z, sizeof(z)));
  }
  return MTB_OK;
}

// Self-test of the give-up path every tensor-core kernel shares: a CTA allocates tensor memory,
// then one thread waits (with the given limit) on an mbarrier that nothing will ever complete.
// The wait runs out, the waiter records `code` in the status word and raises the CTA's abort flag,
// and the kernel tears down like the real ones: tensor memory is freed, the CTA exits.
namespace {
__global__ void __launch_bounds__(64, 1) tc_wait_selftest_kernel(long long limit_cycles, int code) {
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), 32);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 0 && lane == 0) mbar_wait_limit(smem_u32(&bar), 0, &abort_flag, code, limit_cycles);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_slot, 32);
  }
}
}  // namespace

MTB_API int mtb_tc_wait_selftest(long long limit_cycles, int code, void* stream) {
  MTB_REQUIRE(limit_cycles > 0 && limit_cycles <= 200000000LL && code != 0, "tc_wait_selftest: limit must be 1..2e8 cycles and code non-zero");
  tc_wait_selftest_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(limit_cycles, code);
  MTB_LAUNCH_CHECK("tc_wait_selftest_kernel");
  return MTB_OK;
}

bool mtb_tc_gemm_supported(int m, int n, int k, const float* a, int trans_a, const float* b, int trans_b, const float* c) {
  if (getenv("MTB_DISABLE_TC")) return false;
  if (!al16(a) || !al16(b) || !al16(c)) return false;
  if (m < 32 || n < 8 || k < 32) return false;
  if (k % 4) return false;                 // K-major pitches
  if (trans_a && m % 4) return false;      // A stored [K][M]
  if (!trans_b && n % 4) return false;     // B stored [K][N]
  return true;
}

int mtb_tc_gemm_f32(int m, int n, int k, const float* a, int trans_a, const float* b, int trans_b, const float* bias, int relu, float* c,
                    void* stream) {
  CUtensorMap mapA, mapB;
  int bn = pick_bn_for(n, m);
  int rc;
  if (!trans_a) rc = tc::encode_tiled_2d(&mapA, a, m, k, k, 32, 128);
  else rc = tc::encode_tiled_2d(&mapA, a, k, m, m, 32, 32, true);
  if (rc) return rc;
  if (trans_b) rc = tc::encode_tiled_2d(&mapB, b, n, k, k, 32, bn);
  else rc = tc::encode_tiled_2d(&mapB, b, k, n, n, 32, 32, true);
  if (rc) return rc;
  GemmParams p{};
  p.splits = 1; p.kb_per_split = (k + 31) / 32;
  p.M = m; p.N = n; p.num_kb = (k + 31) / 32;
  p.m_tiles = (m + 127) / 128; p.n_tiles = (n + bn - 1) / bn;
  p.out = c; p.ldo = n; p.bias = bias; p.relu = relu;
  p.KH = 1; p.KW = 1; p.cchunks = p.num_kb;
  cudaStream_t st = (cudaStream_t)stream;
  if (!trans_a && trans_b) return launch_tc_bn<A_KMAJOR, B_KMAJOR>(bn, mapA, mapB, p, st);
  if (!trans_a && !trans_b) return launch_tc_bn<A_KMAJOR, B_MNMAJOR>(bn, mapA, mapB, p, st);
  if (trans_a && trans_b) return launch_tc_bn<A_MNMAJOR, B_KMAJOR>(bn, mapA, mapB, p, st);
  return launch_tc_bn<A_MNMAJOR, B_MNMAJOR>(bn, mapA, mapB, p, st);
}

bool mtb_tc_conv2d_forward_supported(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* x,
                                     const float* wt, const float* y) {
  if (getenv("MTB_DISABLE_TC")) return false;
  if (!al16(x) || !al16(wt) || !al16(y)) return false;
  if (cin % 32 || cout % 4) return false;
  if (sh > 8 || sw > 8 || ph > 100 || pw > 100 || kh > 32 || kw > 32) return false;
  if ((long long)n * h * w * cin * 4 < kMinIm2colBytes) return false;
  return true;
}

// stats / stats_rows (both may be NULL): when given and the shape allows, the kernel also writes partial
// rows [rows][3][cout] of per-channel (count, mean, M2) of y and *stats_rows receives their number;
// *stats_rows == 0 means this launch did not produce statistics.
int mtb_tc_conv2d_forward_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* x,
                              const float* wt, const float* bias, float* y, int relu, void* workspace, long long workspace_bytes, void* stream,
                              float* stats, int* stats_rows) {
  const int oh = (h + 2 * ph - kh) / sh + 1, ow = (w + 2 * pw - kw) / sw + 1;
  const long long M = (long long)n * oh * ow, K = (long long)kh * kw * cin;
  const bool rows_path = row_conv_plan(n, h, w, kh, kw, sh, sw, ph, pw, cin, cout, pick_bn_for(cout, M)).ok;
  GemmPlan gp = plan_gemm(cout, M, (int)(K / 32), !rows_path && workspace != nullptr);
  if (split_partial_bytes(gp, M, cout) > workspace_bytes) gp = GemmPlan{pick_bn_for(cout, M), 1, (int)(K / 32)};
  const int bn = rows_path ? pick_bn_for(cout, M) : gp.bn;
  if (stats_rows) *stats_rows = 0;
  const bool want_stats = stats && stats_rows && !relu && cout % 32 == 0 && (!bias || al16(bias)) && !getenv("MTB_DISABLE_CONV_STATS");
  CUtensorMap mapA, mapB;
  int rc = tc::encode_tiled_2d(&mapB, wt, cout, K, K, 32, bn);
  if (rc) return rc;
  const RowConvPlan plan = row_conv_plan(n, h, w, kh, kw, sh, sw, ph, pw, cin, cout, bn);
  if (plan.ok) {
    if (want_stats) *stats_rows = row_conv_stats_rows(plan, (long long)n * plan.Hv * plan.Wp, cout, bn);
    return run_row_conv<B_KMAJOR>(plan, bn, n, h, w, cin, kh, kw, ph, pw, cout, x, mapB, nullptr, bias, nullptr, relu, y, (cudaStream_t)stream,
                                  want_stats ? stats : nullptr);
  }
  rc = tc::encode_im2col_4d(&mapA, x, n, h, w, cin, -pw, -ph, pw - (kw - 1), ph - (kh - 1), sw, sh, 32, 128);
  if (rc) return rc;
  GemmParams p{};
  p.M = (int)M; p.N = cout; p.num_kb = (int)(K / 32);
  p.m_tiles = (int)((M + 127) / 128); p.n_tiles = (cout + bn - 1) / bn;
  p.out = y; p.ldo = cout; p.bias = bias; p.relu = relu;
  p.OW = ow; p.OH = oh; p.SW = sw; p.SH = sh; p.PW = pw; p.PH = ph; p.KW = kw; p.KH = kh; p.cchunks = cin / 32;
  p.splits = gp.splits; p.kb_per_split = gp.kb_per_split; p.partial = (float*)workspace;
  // short reductions (1x1 shortcuts) leave the epilogue no main loop to hide the statistics behind
  // ... unless the output is small: then BatchNorm's own pass is all launch latency, and the epilogue is cheaper
  // (measured on the three 1x1 shortcuts of ResNet-18: 1.782 -> 1.770 ms per step at 64 images, but
  // 6.37 -> 6.41 ms at 512, where their outputs are 17 to 67 MB)
  const bool small_output = (long long)M * cout * 4 <= (12ll << 20);
  if (want_stats && (p.num_kb >= 16 || small_output)) {
    p.stats = stats;
    *stats_rows = gp.splits > 1 ? p.m_tiles * 4 : stats_rows_for(p.m_tiles * p.n_tiles, p.n_tiles);
    cudaStream_t st = (cudaStream_t)stream;
    if (bn == 64) return launch_tc<64, A_IM2COL, B_KMAJOR, true>(mapA, mapB, p, st);
    if (bn == 128) return launch_tc<128, A_IM2COL, B_KMAJOR, true>(mapA, mapB, p, st);
    return launch_tc<256, A_IM2COL, B_KMAJOR, true>(mapA, mapB, p, st);
  }
  return launch_tc_bn<A_IM2COL, B_KMAJOR>(bn, mapA, mapB, p, (cudaStream_t)stream);
}

bool mtb_tc_conv2d_dgrad_supported(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* dy,
                                   const float* wt, const float* dx) {
  if (getenv("MTB_DISABLE_TC")) return false;
  if (!al16(dy) || !al16(wt) || !al16(dx)) return false;
  if (cout % 32 || cin % 4) return false;
  if (kh * kw > 64 || sh > 8 || sw > 8 || ph > 64 || pw > 64) return false;
  const int oh = (h + 2 * ph - kh) / sh + 1, ow = (w + 2 * pw - kw) / sw + 1;
  if ((long long)n * oh * ow * cout * 4 < kMinIm2colBytes) return false;
  return true;
}

// Data gradient.  For stride 1 this is a convolution of dY with the filter rotated by 180
// degrees.  For stride s the input pixels fall into s*s residue classes; pixels of class (a, b)
// only see the taps kh = a (mod s), kw = b (mod s), and over the class's own (coarser) grid
// that is again a stride-1 convolution of dY with that sub-filter.  Each class is one launch of
// the implicit-GEMM kernel: dY plays the activation role (im2col-mode loads with zero fill
// beyond the edges), the weights are read in place as an MN-major operand (for one tap, rows
// are output channels = the reduction index, columns are input channels), and the epilogue
// scatters rows to the class's pixels.  Classes without taps (stride larger than the filter)
// receive zeros.  No atomics; every element of dX is written exactly once.
// addend (may be NULL): dx = dgrad + addend.  Fused into the epilogue on the row-staged path; the
// other paths write dgrad and add afterwards.
int mtb_tc_conv2d_dgrad_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* dy,
                            const float* wt, const float* addend, float* dx, void* workspace, long long workspace_bytes, void* stream) {
  const int oh = (h + 2 * ph - kh) / sh + 1, ow = (w + 2 * pw - kw) / sw + 1;
  // one tile width for all residue classes (the weight tensor map is shared): the one the cost model picks
  // for a class-sized problem
  const long long class_rows = (long long)n * h * w / (sh * sw);
  const bool rows_path = row_conv_plan(n, h, w, kh, kw, sh, sw, ph, pw, cout, cin, pick_bn_for(cin, class_rows)).ok;
  const int class_kb = ((kh + sh - 1) / sh) * ((kw + sw - 1) / sw) * (cout / 32);
  const int bn = rows_path ? pick_bn_for(cin, class_rows) : plan_gemm(cin, class_rows, class_kb, workspace != nullptr).bn;
  cudaStream_t st = (cudaStream_t)stream;
  CUtensorMap mapB;
  int rc = tc::encode_tiled_2d(&mapB, wt, cout, (long long)kh * kw * cin, (long long)kh * kw * cin, 32, 32, true);
  if (rc) return rc;
  const RowConvPlan plan = row_conv_plan(n, h, w, kh, kw, sh, sw, ph, pw, cout, cin, bn);
  if (plan.ok) {
    // stride 1: dX = dY convolved with the filter rotated by 180 degrees, same padding
    int tap_x[64];
    for (int jh = 0; jh < kh; ++jh)
      for (int jw = 0; jw < kw; ++jw) tap_x[jh * kw + jw] = ((kh - 1 - jh) * kw + (kw - 1 - jw)) * cin;
    return run_row_conv<B_MNMAJOR>(plan, bn, n, h, w, cout, kh, kw, ph, pw, cin, dy, mapB, tap_x, nullptr, addend, 0, dx, st);
  }
  struct Axis { int taps, start, count, lower, upper; };
  auto axis = [](int a, int size, int osize, int k, int s, int pad) {
    Axis r{};
    r.taps = a < k ? (k - a + s - 1) / s : 0;
    r.start = (((a - pad) % s) + s) % s;
    r.count = r.start < size ? (size - r.start + s - 1) / s : 0;
    const int c0 = (r.start + pad - a) / s;
    r.lower = c0 - (r.taps - 1);
    r.upper = r.count - osize + r.lower;
    return r;
  };
  bool need_zero = false;
  for (int a = 0; a < sh; ++a)
    for (int b = 0; b < sw; ++b) {
      Axis ah = axis(a, h, oh, kh, sh, ph), aw = axis(b, w, ow, kw, sw, pw);
      if (ah.count > 0 && aw.count > 0 && (ah.taps == 0 || aw.taps == 0)) need_zero = true;
    }
  // addend == dx: dx already holds the gradient to add to; every class adds its own pixels in its epilogue
  // and the pixels of classes without taps stay as they are.
  const bool in_place = addend != nullptr && addend == dx;
  if (need_zero && !in_place) MTB_CUDA(cudaMemsetAsync(dx, 0, (size_t)n * h * w * cin * 4, st));
  // The classes write disjoint pixels.  When one class fills only part of the GPU they run side by side on
  // separate lanes (then without split reductions, whose tickets and partials one launch at a time owns).
  int live = 0;
  for (int a = 0; a < sh; ++a)
    for (int b = 0; b < sw; ++b) {
      Axis ah = axis(a, h, oh, kh, sh, ph), aw = axis(b, w, ow, kw, sw, pw);
      if (ah.count > 0 && aw.count > 0 && ah.taps > 0 && aw.taps > 0) ++live;
    }
  const long long class_units = ((class_rows + 127) / 128) * ((cin + bn - 1) / bn);
  const bool side_by_side = live > 1 && class_units < mtb_sm_count() && !getenv("MTB_DGRAD_SERIAL");
  const int lanes = side_by_side ? (live < kMaxLanes ? live : kMaxLanes) : 1;
  cudaStream_t lane_stream[kMaxLanes];
  rc = mtb_fork_lanes(st, lanes, lane_stream);
  if (rc) return rc;
  int launched = 0;
  for (int a = 0; a < sh; ++a) {
    for (int b = 0; b < sw; ++b) {
      Axis ah = axis(a, h, oh, kh, sh, ph), aw = axis(b, w, ow, kw, sw, pw);
      if (ah.count == 0 || aw.count == 0 || ah.taps == 0 || aw.taps == 0) continue;
      cudaStream_t cst = lane_stream[launched++ % lanes];
      CUtensorMap mapA;
      rc = tc::encode_im2col_4d(&mapA, dy, n, oh, ow, cout, aw.lower, ah.lower, aw.upper, ah.upper, 1, 1, 32, 128);
      if (rc) return rc;
      GemmParams p{};
      const long long M = (long long)n * ah.count * aw.count;
      p.M = (int)M; p.N = cin; p.num_kb = ah.taps * aw.taps * (cout / 32);
      GemmPlan gp = plan_gemm(cin, M, p.num_kb, workspace != nullptr && lanes == 1, bn);
      if (split_partial_bytes(gp, M, cin) > workspace_bytes) gp = GemmPlan{bn, 1, p.num_kb};
      p.splits = gp.splits; p.kb_per_split = gp.kb_per_split; p.partial = (float*)workspace;
      p.m_tiles = (int)((M + 127) / 128); p.n_tiles = (cin + bn - 1) / bn;
      p.out = dx; p.ldo = cin; p.bias = nullptr; p.relu = 0;
      p.accumulate = in_place ? 1 : 0;
      p.OW = aw.count; p.OH = ah.count; p.SW = 1; p.SH = 1; p.PW = -aw.lower; p.PH = -ah.lower; p.KW = aw.taps; p.KH = ah.taps;
      p.cchunks = cout / 32;
      p.b_per_tap = 1;
      for (int jh = 0; jh < ah.taps; ++jh)
        for (int jw = 0; jw < aw.taps; ++jw) {
          const int fkh = a + sh * (ah.taps - 1 - jh), fkw = b + sw * (aw.taps - 1 - jw);  // dY offset j <-> filter tap
          p.b_tap_x[jh * aw.taps + jw] = (fkh * kw + fkw) * cin;
        }
      p.o_strided = 1; p.o_Hc = ah.count; p.o_Wc = aw.count; p.o_H = h; p.o_W = w; p.o_h0 = ah.start; p.o_w0 = aw.start; p.o_sh = sh; p.o_sw = sw;
      rc = launch_tc_bn<A_IM2COL, B_MNMAJOR>(bn, mapA, mapB, p, cst);
      if (rc) return rc;
    }
  }
  rc = mtb_join_lanes(st, lanes);
  if (rc) return rc;
  if (addend && !in_place) return mtb_add_f32(dx, addend, dx, (long long)n * h * w * cin, 1.0f, st);
  return MTB_OK;
}

// True when mtb_tc_conv2d_dgrad_f32 with addend == dx (accumulate in place) is available AND is the cheaper
// form: strided convolutions some of whose residue classes have no taps (1x1 with stride 2), where the
// out-of-place form costs a memset, a scattered write and a pass that adds the two tensors.
bool mtb_tc_conv2d_dgrad_in_place(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* dy,
                                  const float* wt, const float* dx) {
  if (!mtb_tc_conv2d_dgrad_supported(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, dy, wt, dx)) return false;
  if (sh * sw == 1 || getenv("MTB_DGRAD_OUT_OF_PLACE")) return false;
  return kh < sh || kw < sw;  // a residue class a >= kh (b >= kw) sees no tap
}

// ------------------------------------------------------------------------------ weight gradient
//
// dW^T[(tap, ci), co] = sum over output pixels m of patch(X)[m, (tap, ci)] * dY[m, co].
// Both operands are "MN-major" in memory (for a fixed pixel, channels are contiguous), so they
// are staged exactly as they lie: the A tile is 4 im2col-mode loads of 32 pixels x 32 channels
// (one per (tap, channel-block)), the B tile BN/32 boxes of 32 pixels x 32 output channels.
// The reduction runs over pixels, which is long (up to N*OH*OW) while the output is small, so
// the pixel range is split across CTAs; each writes an fp32 partial to scratch and a second
// kernel adds the partials in a fixed order and transposes into dW[co][tap][ci].
namespace {

// PB pixels (reduction elements) per stage; one A chunk = PB pixels x 32 channels.
template <int BN, int PB>
struct WCfg {
  static constexpr uint32_t kChunk = PB * 128;
  static constexpr uint32_t kABytes = 4 * kChunk;
  static constexpr uint32_t kBBytes = (BN / 32) * kChunk;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr int kStagesFit = (227 * 1024 - 2048) / kStageBytes;
  static constexpr int kStages = kStagesFit > 6 ? 6 : kStagesFit;
  static constexpr uint32_t kSmemBytes = kStages * kStageBytes + 1024;
  static constexpr uint32_t kTmemCols = 2 * BN;
};

struct WgradParams {
  int Kw;            // KH*KW*Cin: rows of the transposed gradient
  int Cout;
  int chunks;        // Kw / 32
  int cchunks;       // Cin / 32
  int m_tiles, n_tiles, splits;
  int kb_total;      // ceil(pixels / PB)
  int kb_per_split;
  int OW, OH, SW, SH, PW, PH, KW;
  float* partial;    // [splits][Kw][Cout]
};

template <int BN, int PB>
__global__ void __launch_bounds__(192, 1)
tc_wgrad_kernel(const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapDY, const WgradParams p) {
  using C = WCfg<BN, PB>;
  constexpr int STAGES = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_full[8], bar_empty[8], bar_tfull[2], bar_tempty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_tfull[b]), 1);
      mbar_init(smem_u32(&bar_tempty[b]), 4);  // one arrival per epilogue warp
    }
    abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  const int units = p.m_tiles * p.n_tiles * p.splits;
  volatile int* abort_ptr = &abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tensormap(&mapX);
      prefetch_tensormap(&mapDY);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
        const int split = unit % p.splits, tile = unit / p.splits;
        const int m_tile = tile / p.n_tiles, n0 = (tile % p.n_tiles) * BN;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = kb0 + p.kb_per_split < p.kb_total ? kb0 + p.kb_per_split : p.kb_total;
        int valid = p.chunks - m_tile * 4;
        if (valid > 4) valid = 4;
        const uint32_t bytes = (uint32_t)valid * C::kChunk + C::kBBytes;
        int q_c[4], q_kw[4], q_kh[4];
        for (int q = 0; q < 4; ++q) {
          const int chunk = m_tile * 4 + (q < valid ? q : 0);
          const int tap = chunk / p.cchunks;
          q_c[q] = (chunk - tap * p.cchunks) * 32;
          q_kh[q] = tap / p.KW;
          q_kw[q] = tap - q_kh[q] * p.KW;
        }
        // first pixel of the range, then advanced by PB pixels per block without divisions
        int m = kb0 * PB;
        int ow = m % p.OW, tq = m / p.OW;
        int oh = tq % p.OH, pn_ = tq / p.OH;
        for (int kb = kb0; kb < kb1; ++kb, m += PB) {
          if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abort_ptr, 11)) { ok = false; break; }
          const uint32_t full = smem_u32(&bar_full[stage]);
          mbar_expect_tx(full, bytes);
          const uint32_t a_dst = smem_base + stage * C::kStageBytes, b_dst = a_dst + C::kABytes;
          const int pw_ = ow * p.SW - p.PW, ph_ = oh * p.SH - p.PH;
#pragma unroll
          for (int q = 0; q < 4; ++q)
            if (q < valid) tma_load_im2col_4d(a_dst + q * C::kChunk, &mapX, full, q_c[q], pw_, ph_, pn_, (uint16_t)q_kw[q], (uint16_t)q_kh[q]);
#pragma unroll
          for (int j = 0; j < BN / 32; ++j) tma_load_2d(b_dst + j * C::kChunk, &mapDY, full, n0 + 32 * j, m);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          ow += PB;
          while (ow >= p.OW) {
            ow -= p.OW;
            if (++oh == p.OH) { oh = 0; ++pn_; }
          }
        }
      }
    }
  } else if (warp == 1) {
    // converged warp, elected issue (see tc_gemm_kernel)
    constexpr uint32_t idesc = idesc_tf32(128, BN, 1, 1);
    constexpr uint32_t hi = desc_hi_mnmajor();
    constexpr uint32_t step = 1024u >> 4;
    const uint32_t a_lo0 = desc_lo_mnmajor(smem_base, C::kChunk), b_lo0 = desc_lo_mnmajor(smem_base + C::kABytes, C::kChunk);
    int stage = 0;
    uint32_t phase = 0;
    int t = 0;
    bool ok = true;
    for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x, ++t) {
      const int split = unit % p.splits;
      const int kb0 = split * p.kb_per_split;
      const int kb1 = kb0 + p.kb_per_split < p.kb_total ? kb0 + p.kb_per_split : p.kb_total;
      const int buf = t & 1;
      const uint32_t use = (uint32_t)(t >> 1);
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_tempty[buf]), (use & 1u) ^ 1u, abort_ptr, 12));
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + buf * BN;
      uint32_t acc = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_full[stage]), phase, abort_ptr, 13));
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_lo = a_lo0 + stage * (C::kStageBytes >> 4), b_lo = b_lo0 + stage * (C::kStageBytes >> 4);
        if (elect_one()) {
          mma_tf32_words(d_tmem, a_lo, hi, b_lo, hi, idesc, acc);
#pragma unroll
          for (int kk = 1; kk < PB / 8; ++kk) mma_tf32_words(d_tmem, a_lo + kk * step, hi, b_lo + kk * step, hi, idesc, 1u);
          mma_commit(smem_u32(&bar_empty[stage]));
        }
        __syncwarp();
        acc = 1u;
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
      if (ok && elect_one()) mma_commit(smem_u32(&bar_tfull[buf]));
      __syncwarp();
    }
  } else {
    const int quarter = warp & 3;
    int t = 0;
    const bool wide_ok = (p.Cout % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.partial) & 31u) == 0);  // 32-byte stores
    for (int unit = blockIdx.x; unit < units; unit += gridDim.x, ++t) {
      const int split = unit % p.splits, tile = unit / p.splits;
      const int m_tile = tile / p.n_tiles, n0 = (tile % p.n_tiles) * BN;
      const int kb0 = split * p.kb_per_split;
      const bool empty_unit = kb0 >= p.kb_total;  // cannot happen with the host's split choice; kept for safety
      const int buf = t & 1;
      const uint32_t use = (uint32_t)(t >> 1);
      // one lane polls (128 threads spinning on the barrier slow the other roles' barrier traffic down)
      bool ok = lane != 0 || mbar_wait(smem_u32(&bar_tfull[buf]), use & 1u, abort_ptr, 14);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = m_tile * 128 + quarter * 32 + lane;
      float* orow = p.partial + ((long long)split * p.Kw + row) * p.Cout;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c0), r);
        tmem_ld_wait();
        const int col0 = n0 + c0;
        if (row < p.Kw && col0 < p.Cout) {
          if (col0 + 32 <= p.Cout) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
              float4 u = make_float4(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]), __uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
              if (empty_unit) v = u = make_float4(0.f, 0.f, 0.f, 0.f);
              st_row8(orow + col0 + j, v, u, wide_ok);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.Cout) orow[col0 + j] = empty_unit ? 0.f : __uint_as_float(r[j]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[buf]));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// dw[co][r] = sum_s partial[s][r][co]: a CTA takes 32 rows x 128 output channels, reads float4
// along co (splits added in index order), transposes through shared memory and writes 128-byte
// runs along r.
__global__ void __launch_bounds__(1024) wgrad_reduce_transpose_kernel(const float* __restrict__ partial, float* __restrict__ dw, int Kw, int Cout,
                                                                       int splits) {
  __shared__ float tile[128][33];
  const int r0 = blockIdx.x * 32, c0 = blockIdx.y * 128;
  const long long plane = (long long)Kw * Cout;
  {
    const int r = r0 + threadIdx.y, c = c0 + 4 * threadIdx.x;
    float4 s0 = make_float4(0.f, 0.f, 0.f, 0.f), s1 = s0;
    if (r < Kw && c < Cout) {  // Cout % 4 == 0 on this path, so the four channels are in range together
      const float* q = partial + (long long)r * Cout + c;
      int z = 0;
      for (; z + 1 < splits; z += 2) {  // two independent loads in flight; the grouping is fixed
        const float4 a = *reinterpret_cast<const float4*>(q + z * plane);
        const float4 b = *reinterpret_cast<const float4*>(q + (z + 1) * plane);
        s0.x += a.x; s0.y += a.y; s0.z += a.z; s0.w += a.w;
        s1.x += b.x; s1.y += b.y; s1.z += b.z; s1.w += b.w;
      }
      if (z < splits) {
        const float4 a = *reinterpret_cast<const float4*>(q + z * plane);
        s0.x += a.x; s0.y += a.y; s0.z += a.z; s0.w += a.w;
      }
    }
    tile[4 * threadIdx.x + 0][threadIdx.y] = s0.x + s1.x;
    tile[4 * threadIdx.x + 1][threadIdx.y] = s0.y + s1.y;
    tile[4 * threadIdx.x + 2][threadIdx.y] = s0.z + s1.z;
    tile[4 * threadIdx.x + 3][threadIdx.y] = s0.w + s1.w;
  }
  __syncthreads();
  const int r = r0 + threadIdx.x;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int cc = threadIdx.y + 32 * k, c = c0 + cc;
    if (r < Kw && c < Cout) dw[(long long)c * Kw + r] = tile[cc][threadIdx.x];
  }
}

struct WgradPlan {
  int bn, pb, m_tiles, n_tiles, splits, kb_total, kb_per_split;
  long long Kw, pixels;
};

WgradPlan wgrad_plan(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout) {
  WgradPlan q;
  const int oh = (h + 2 * ph - kh) / sh + 1, ow = (w + 2 * pw - kw) / sw + 1;
  q.pixels = (long long)n * oh * ow;
  q.Kw = (long long)kh * kw * cin;
  q.bn = pick_bn(cout);
  q.m_tiles = (int)((q.Kw + 127) / 128);
  q.n_tiles = (cout + q.bn - 1) / q.bn;
  // An im2col-mode load costs roughly the same whatever its size (measured: 4 loads of 32 pixels per
  // stage ran at 100 TFLOP/s, 4 loads of 64 pixels at 169), so stages hold 64 pixels even where only
  // two stages then fit (BN = 256: 239 -> 290 TFLOP/s).
  q.pb = 64;
  q.kb_total = (int)((q.pixels + q.pb - 1) / q.pb);
  const int tiles = q.m_tiles * q.n_tiles;
  // as many splits as still fit the GPU in ONE wave (rounding up instead left a second, nearly empty wave:
  // 18 tiles x 9 splits = 162 units on 148 SMs ran 117 us, 8 splits run one wave)
  int splits = mtb_sm_count() / tiles;
  const int max_splits = (q.kb_total + 3) / 4;  // at least 4 reduction blocks per CTA
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  q.kb_per_split = (q.kb_total + splits - 1) / splits;
  q.splits = (q.kb_total + q.kb_per_split - 1) / q.kb_per_split;  // no empty split
  return q;
}

}  // namespace

// Which kernel family each of forward / data gradient / weight gradient would take for a shape
// (pointers assumed 16-byte aligned), and, for the row-staged kernels, how their shared and tensor
// memory is laid out against the furthest byte their copies write and their descriptors read.
// Host code only: callable without a device (the SM count then defaults to 148).
//   out[0..2]   path of forward, dgrad, wgrad: 0 CUDA-core, 1 im2col tcgen05, 2 row-staged tcgen05
//   out[3..9]   forward, row-staged: dynamic smem bytes, activation stage bytes, last byte written by
//               the row copies, last byte read through a descriptor, TMEM columns, tiles per item,
//               1 if the filter is resident
//   out[10..16] the same for dgrad
//   out[17..24] wgrad, row-staged: dynamic smem bytes, X panel bytes, last byte written, last byte
//               read, dY panel bytes, last byte written, last byte read, TMEM columns
MTB_API int mtb_conv2d_plan_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, int* out) {
  MTB_REQUIRE(out && n > 0 && cin > 0 && cout > 0 && h > 0 && w > 0 && kh > 0 && kw > 0 && sh > 0 && sw > 0, "conv2d_plan: bad arguments");
  for (int i = 0; i < 25; ++i) out[i] = 0;
  const float* al = reinterpret_cast<const float*>(uintptr_t(256));
  const int oh = (h + 2 * ph - kh) / sh + 1, ow = (w + 2 * pw - kw) / sw + 1;
  if (oh <= 0 || ow <= 0) return MTB_OK;
  auto describe = [&](int slot, int kc, int nout, long long rows) {
    const int bn = pick_bn_for(nout, rows);
    const RowConvPlan q = row_conv_plan(n, h, w, kh, kw, sh, sw, ph, pw, kc, nout, bn);
    if (!q.ok) return false;
    const long long span = 128LL * q.mt;
    out[slot + 0] = (int)q.smem_bytes;
    out[slot + 1] = (int)q.a_stage_bytes;
    out[slot + 2] = (int)(kRowLead + (long long)q.nr_max * q.Wp * 128);
    out[slot + 3] = (int)(kRowLead + ((q.Wp - 1) + (span - 1) + (long long)(kh - 1) * q.Wp + (kw - 1) - pw + 1) * 128);
    out[slot + 4] = 2 * q.mt * bn;
    out[slot + 5] = q.mt;
    out[slot + 6] = q.resident;
    return true;
  };
  if (mtb_tc_conv2d_forward_supported(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, al, al, al))
    out[0] = describe(3, cin, cout, (long long)n * oh * ow) ? 2 : 1;
  if (mtb_tc_conv2d_dgrad_supported(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, al, al, al))
    out[1] = describe(10, cout, cin, (long long)n * h * w / (sh * sw)) ? 2 : 1;
  if (mtb_tc_conv2d_wgrad_supported(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, al, al, al)) {
    const WgradRowsPlan q = wgrad_rows_plan(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout);
    out[2] = q.ok ? 2 : 1;
    if (q.ok) {
      const int nr_y = (q.Wp - 1 + kWgRowsPB - 1) / q.Wp + 1, nr_x = nr_y + 2 * ph;
      out[17] = (int)q.smem_bytes;
      out[18] = (int)q.x_panel_bytes;
      out[19] = (int)(kRowLead + (long long)nr_x * q.Wp * 128);
      out[20] = (int)(kRowLead + ((q.Wp - 1) - pw + (long long)(kh - 1) * q.Wp + 4 * q.n_kwg - 1 + (kWgRowsPB - 1) + 1) * 128);
      out[21] = (int)q.y_panel_bytes;
      out[22] = (int)((long long)nr_y * q.Wp * 128);
      out[23] = (int)(((q.Wp - 1) + (kWgRowsPB - 1) + 1) * 128);
      out[24] = kh * q.n_kwg * q.ncc_g * q.bn;
    }
  }
  return MTB_OK;
}

long long mtb_tc_conv2d_workspace_bytes(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout) {
  if (cin % 32) return 0;
  WgradPlan q = wgrad_plan(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout);
  long long bytes = (long long)q.splits * q.Kw * cout * 4 + 256;
  // forward / data gradient with a split reduction: at most one unit per SM, each a 128 x 256 fp32 partial
  const long long split_bytes = (long long)mtb_sm_count() * 128 * 256 * 4;
  if (split_bytes > bytes) bytes = split_bytes;
  const WgradRowsPlan rq = wgrad_rows_plan(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout);
  if (rq.ok) {
    const long long b2 = (long long)rq.splits * q.Kw * cout * 4 + 256;
    if (b2 > bytes) bytes = b2;
  }
  return bytes;
}

bool mtb_tc_conv2d_wgrad_supported(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* x,
                                   const float* dy, const float* dw) {
  if (getenv("MTB_DISABLE_TC")) return false;
  if (!al16(x) || !al16(dy) || !al16(dw)) return false;
  if (cin % 32 || cout % 4) return false;
  if (sh > 8 || sw > 8 || ph > 100 || pw > 100 || kh > 32 || kw > 32) return false;
  if ((long long)n * h * w * cin * 4 < kMinIm2colBytes) return false;
  return true;
}

int mtb_tc_conv2d_wgrad_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* x,
                            const float* dy, float* dw, void* workspace, long long workspace_bytes, void* stream) {
  const int oh = (h + 2 * ph - kh) / sh + 1, ow = (w + 2 * pw - kw) / sw + 1;
  const WgradRowsPlan rq = wgrad_rows_plan(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout);
  if (rq.ok) {
    MTB_REQUIRE(workspace && workspace_bytes >= (long long)rq.splits * kh * kw * cin * cout * 4, "conv2d_wgrad: workspace too small");
    return run_wgrad_rows(rq, n, cin, h, w, kh, kw, ph, pw, cout, x, dy, dw, (float*)workspace, (cudaStream_t)stream);
  }
  WgradPlan q = wgrad_plan(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout);
  MTB_REQUIRE(workspace && workspace_bytes >= (long long)q.splits * q.Kw * cout * 4, "conv2d_wgrad: workspace too small");
  CUtensorMap mapX, mapDY;
  int rc = tc::encode_im2col_4d(&mapX, x, n, h, w, cin, -pw, -ph, pw - (kw - 1), ph - (kh - 1), sw, sh, 32, q.pb, true);
  if (rc) return rc;
  rc = tc::encode_tiled_2d(&mapDY, dy, q.pixels, cout, cout, 32, q.pb, true);
  if (rc) return rc;
  WgradParams p{};
  p.Kw = (int)q.Kw; p.Cout = cout; p.chunks = (int)(q.Kw / 32); p.cchunks = cin / 32;
  p.m_tiles = q.m_tiles; p.n_tiles = q.n_tiles; p.splits = q.splits; p.kb_total = q.kb_total; p.kb_per_split = q.kb_per_split;
  p.OW = ow; p.OH = oh; p.SW = sw; p.SH = sh; p.PW = pw; p.PH = ph; p.KW = kw;
  p.partial = (float*)workspace;
  cudaStream_t st = (cudaStream_t)stream;
  const int units = q.m_tiles * q.n_tiles * q.splits;
  const int grid = units < mtb_sm_count() ? units : mtb_sm_count();
#define MTB_LAUNCH_WGRAD(BN_, PB_)                                                                                      \
  do {                                                                                                                  \
    static unsigned long long configured = 0;                                                                           \
    if (int rc_ = mtb_opt_in_smem((const void*)tc_wgrad_kernel<BN_, PB_>, (int)WCfg<BN_, PB_>::kSmemBytes, &configured)) \
      return rc_;                                                                                                       \
    tc_wgrad_kernel<BN_, PB_><<<grid, 192, WCfg<BN_, PB_>::kSmemBytes, st>>>(mapX, mapDY, p);                           \
  } while (0)
  if (q.bn == 64) MTB_LAUNCH_WGRAD(64, 64);
  else if (q.bn == 128) MTB_LAUNCH_WGRAD(128, 64);
  else MTB_LAUNCH_WGRAD(256, 64);
#undef MTB_LAUNCH_WGRAD
  MTB_LAUNCH_CHECK("tc_wgrad_kernel");
  dim3 rgrid((unsigned)((q.Kw + 31) / 32), (unsigned)((cout + 127) / 128));
  wgrad_reduce_transpose_kernel<<<rgrid, dim3(32, 32), 0, st>>>((const float*)workspace, dw, (int)q.Kw, cout, q.splits);
  MTB_LAUNCH_CHECK("wgrad_reduce_transpose_kernel");
  return MTB_OK;
}
