// Stride-1 "same" convolution (KH = 2*PH+1, KW = 2*PW+1) on tcgen05 with the activation staged
// ONCE per tile instead of once per filter tap.
//
// The im2col-mode kernel copies every input pixel into shared memory KH*KW times (once per
// tap).  Shared memory moves 128 B per cycle per SM in total, shared between the copy engine
// writing tiles and the tensor core reading them, and for narrow layers that traffic, not the
// MMA rate, bounds the kernel.  Here the activation is laid out in shared memory as whole image
// rows, each padded to Wp = W + 2*PW pixels with the zeros the copy engine fills in beyond the
// edges; consecutive rows follow each other without gaps, and images are separated by PH rows
// of zeros.  In that "padded linear" space the pixel a tap (kh, kw) needs for output position q
// is simply position q + (kh-PH)*Wp + (kw-PW), so the A operand of every tap is the SAME
// shared-memory tile read through a descriptor whose start address is shifted by whole
// 128-byte rows (the 128-byte swizzle is a function of the address bits, so a row shift keeps
// it consistent).  A tile is 128 consecutive positions; positions that fall on padding columns
// or separator rows are computed and thrown away (W*H / (Wp*(H+PH)) of the work is useful,
// 91 % for 32x32 images and 3x3 filters).
//
// Loop nest per tile: for each block of 32 reduction channels { stage the rows once (one copy
// per image row); for each tap { stage the BN x 32 weight tile; 4 MMAs of K = 8 } }.
// Roles, barriers, bounded waits and the TMEM double buffer are those of tc_gemm_kernel.
#pragma once

namespace {
using namespace tc;

struct RowConvParams {
  long long Q;             // positions: N * Hv * Wp
  int Wp, Hv, H, W, PH, PW, KH, KW;
  int cchunks;             // reduction channels / 32
  int kc_total;            // reduction channels (pitch of one tap in the K-major weight matrix)
  int N;                   // output channels
  int m_tiles, n_tiles;
  uint32_t a_stage_bytes;  // multiple of 1024; rows start kRowLead bytes into the stage
  int b_stages;            // weight ring depth
  int tps;                 // filter taps per weight stage
  int resident;            // the whole filter (all taps, all channel blocks) stays in shared memory
  float* out;
  long long ldo;
  const float* bias;
  const float* addend;     // optional [same shape as out]: out = conv + addend (gradient accumulation)
  int relu;
  int issuers;             // issuing warps at work (1 or 2)
  int b_tap_x[64];         // MN-major B only: first column of tap j in the weight matrix
  // STATS kernels only: partial rows [(blockIdx.x / n_tiles) * 4 + epilogue warp][3][N] of per-channel
  // (count, mean, M2) over the pixels this CTA produced (grid is a multiple of n_tiles)
  float* stats;
};

constexpr uint32_t kRowLead = 1024;  // room for the left-most tap of the first position to reach back
constexpr int kRowAStages = 2;
constexpr int kRowIssuers = 2;                        // warps 1..2 issue MMAs, on alternating tiles
constexpr int kRowThreads = 32 * (1 + kRowIssuers + 4);  // producer, issuers, four epilogue warps

// Why a weight stage holds several taps: one producer/consumer hand-over through a pair of
// mbarriers costs the issuing thread about 300-400 cycles that do not overlap with tensor-core
// work, and a tcgen05.mma takes ~45 cycles to issue whatever its width, so a stage of 4 narrow
// MMAs (192 cycles of work at N = 64) leaves the tensor core idle most of the time.  With all
// nine taps of a 3x3 filter in one stage (36 MMAs) the hand-over is amortised.
// MT = tiles of 128 positions per work item.  With streamed weights two tiles share every weight
// stage (two accumulators), which halves the L2 -> shared-memory weight traffic per MMA; that traffic,
// at ~47 B/cycle/SM, is what bounds the 128-channel layers.
template <int BN, int BMODE, int FK, int MT, bool STATS>
__global__ void __launch_bounds__(kRowThreads, 1)
tc_conv_rows_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const RowConvParams p) {
  constexpr uint32_t kTapBytes = BN * 128;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_afull[kRowAStages], bar_aempty[kRowAStages], bar_bfull[8], bar_bempty[8], bar_tfull[2], bar_tempty[2], bar_bres;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ int tiles_seen;  // tiles of this CTA whose every stage an issuing warp has seen filled

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t b_base = smem_base + kRowAStages * p.a_stage_bytes;
  const uint32_t b_stage_bytes = (uint32_t)p.tps * kTapBytes;
  const int BST = p.b_stages;

  // The shifted reads of the first and last positions of a tile reach a few rows outside what
  // the copies of that tile wrote; those rows only feed discarded outputs, but they must hold
  // finite numbers for nothing else, so the lead and the tail of every stage start as zeros.
  for (uint32_t i = threadIdx.x; i < kRowAStages * p.a_stage_bytes / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(smem_raw + (smem_base - smem_u32(smem_raw)))[i] = make_uint4(0, 0, 0, 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRowAStages; ++s) {
      mbar_init(smem_u32(&bar_afull[s]), 1);
      mbar_init(smem_u32(&bar_aempty[s]), 1);
    }
    for (int s = 0; s < 8; ++s) {
      mbar_init(smem_u32(&bar_bfull[s]), 1);
      mbar_init(smem_u32(&bar_bempty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_tfull[b]), 1);
      mbar_init(smem_u32(&bar_tempty[b]), 4);  // one arrival per epilogue warp
    }
    mbar_init(smem_u32(&bar_bres), 1);
    abort_flag = 0;
    tiles_seen = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), 2 * MT * BN);
    tmem_relinquish();
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  const int tiles = ((p.m_tiles + MT - 1) / MT) * p.n_tiles;  // work items
  const int taps = p.KH * p.KW;
  volatile int* abort_ptr = &abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&mapA);
      prefetch_tensormap(&mapB);
      int as = 0, bs = 0;
      uint32_t aphase = 0, bphase = 0;
      bool ok = true;
      const uint32_t row_bytes = (uint32_t)p.Wp * 128u;
      if (p.resident && blockIdx.x < tiles) {
        // one output-channel tile in all: every (channel block, tap) weight tile is fetched once
        const uint32_t bres = smem_u32(&bar_bres);
        mbar_expect_tx(bres, (uint32_t)(p.cchunks * taps) * kTapBytes);
        uint32_t b_dst = b_base;
        for (int cc = 0; cc < p.cchunks; ++cc)
          for (int tap = 0; tap < taps; ++tap, b_dst += kTapBytes) {
            if (BMODE == B_KMAJOR) {
              tma_load_2d(b_dst, &mapB, bres, tap * p.kc_total + cc * 32, 0);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 32; ++j) tma_load_2d(b_dst + j * 4096, &mapB, bres, p.b_tap_x[tap] + 32 * j, cc * 32);
            }
          }
      }
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        const int q0 = (tile / p.n_tiles) * (128 * MT);  // positions fit 31 bits (checked on the host)
        const int n0 = (tile % p.n_tiles) * BN;
        const int v_lo = q0 / p.Wp - p.PH;
        const int nr = (q0 + 128 * MT - 1) / p.Wp + p.PH - v_lo + 1;
        // first image row: floor division (v_lo is -PH for the very first tile)
        const int img = v_lo >= 0 ? v_lo / p.Hv : -1;
        const int hrow = v_lo - img * p.Hv;
        for (int cc = 0; cc < p.cchunks && ok; ++cc) {
          if (!mbar_wait(smem_u32(&bar_aempty[as]), aphase ^ 1u, abort_ptr, 11)) { ok = false; break; }
          const uint32_t afull = smem_u32(&bar_afull[as]);
          mbar_expect_tx(afull, (uint32_t)nr * row_bytes);
          uint32_t dst = smem_base + as * p.a_stage_bytes + kRowLead;
          int im = img, hr = hrow;
          for (int r = 0; r < nr; ++r, dst += row_bytes) {
            // rows h >= H (separators) and images outside [0, N) are filled with zeros by the copy
            tma_load_4d(dst, &mapA, afull, cc * 32, -p.PW, hr, im);
            if (++hr == p.Hv) { hr = 0; ++im; }
          }
          if (++as == kRowAStages) { as = 0; aphase ^= 1u; }
          for (int tap0 = 0; tap0 < taps && !p.resident; tap0 += p.tps) {
            const int cnt = taps - tap0 < p.tps ? taps - tap0 : p.tps;
            if (!mbar_wait(smem_u32(&bar_bempty[bs]), bphase ^ 1u, abort_ptr, 12)) { ok = false; break; }
            const uint32_t bfull = smem_u32(&bar_bfull[bs]);
            mbar_expect_tx(bfull, (uint32_t)cnt * kTapBytes);
            uint32_t b_dst = b_base + bs * b_stage_bytes;
            for (int tap = tap0; tap < tap0 + cnt; ++tap, b_dst += kTapBytes) {
              if (BMODE == B_KMAJOR) {
                tma_load_2d(b_dst, &mapB, bfull, tap * p.kc_total + cc * 32, n0);
              } else {
#pragma unroll
                for (int j = 0; j < BN / 32; ++j) tma_load_2d(b_dst + j * 4096, &mapB, bfull, p.b_tap_x[tap] + n0 + 32 * j, cc * 32);
              }
            }
            if (++bs == BST) { bs = 0; bphase ^= 1u; }
          }
        }
      }
    }
  } else if (warp <= kRowIssuers) {
    // ------------------------------------------------------------ MMA issuers
    // The whole warp runs the loops converged and one elected lane issues: with warp-uniform
    // control flow the descriptors stay in uniform registers, which roughly halves the cost of
    // issuing a tcgen05.mma compared with a lane-0 branch around everything.
    constexpr uint32_t idesc = idesc_tf32(128, BN, 0, BMODE == B_MNMAJOR ? 1 : 0);
    constexpr uint32_t a_hi = desc_hi_kmajor();
    constexpr uint32_t b_hi = BMODE == B_MNMAJOR ? desc_hi_mnmajor() : desc_hi_kmajor();
    constexpr uint32_t b_step = BMODE == B_MNMAJOR ? (1024u >> 4) : (32u >> 4);
    constexpr uint32_t tap_step = kTapBytes >> 4;
    const uint32_t b_lo0 = BMODE == B_MNMAJOR ? desc_lo_mnmajor(b_base) : desc_lo_kmajor(b_base);
    const uint32_t row_step = (uint32_t)p.Wp * 8u;  // one image row, in 16-byte units (a pixel is 128 B)
    // Two warps issue, each every other tile of this CTA into its own accumulator buffer.  What one warp does
    // between tiles (waiting for the accumulator and the next activation stage, position arithmetic, commits)
    // then runs while the other warp's MMAs keep the tensor pipe busy.  The two never accumulate into the same
    // buffer, so the interleaving of their MMAs in the pipe does not change any sum.  The rings are consumed in
    // tile order, so a warp finds its place in them from the tile's ordinal alone.  A parity wait cannot tell
    // "lap L not yet filled" from "lap L + 1 filled", and the previous lap of a slot may belong to the other
    // warp's tile: so a warp publishes its tile's ordinal once it has seen the tile's last stage filled, and
    // nobody starts waiting on the stages of tile t before tile t - 1 is published (bounded like every wait).
    const int iw = warp - 1;
    const int b_per_cc = p.resident ? 0 : (FK == 3 ? 3 : (taps + p.tps - 1) / p.tps);
    bool ok = true;
    if (p.resident && blockIdx.x < tiles) ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_bres), 0, abort_ptr, 17));
    for (int t = iw; ok && iw < p.issuers; t += p.issuers) {
      const int tile = blockIdx.x + t * (int)gridDim.x;
      if (tile >= tiles) break;
      const int a_g = t * p.cchunks, b_g = a_g * b_per_cc;
      int as = a_g % kRowAStages, bs = b_g % BST;
      int alap = a_g / kRowAStages, blap = b_g / BST;
      const int col = ((tile / p.n_tiles) * (128 * MT)) % p.Wp;
      const int buf = t & 1;
      const uint32_t use = (uint32_t)(t >> 1);
      ok = __all_sync(0xffffffffu, lap_wait(&tiles_seen, t, abort_ptr, 18) &&
                                       mbar_wait(smem_u32(&bar_tempty[buf]), (use & 1u) ^ 1u, abort_ptr, 13));
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + buf * (MT * BN);
      constexpr uint32_t tile_step = 128u * 8u;  // the next tile's positions start 128 pixels (of 8 units) further
      for (int cc = 0; cc < p.cchunks && ok; ++cc) {
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_afull[as]), (uint32_t)alap & 1u, abort_ptr, 14));
        if (!ok) break;
        if (p.resident && cc == p.cchunks - 1) *(volatile int*)&tiles_seen = t + 1;
        tc_fence_after();
        // position q0 of this tile sits PH rows and `col` pixels into the staged rows; tap
        // (kh, kw) reads (kh - PH) rows and (kw - PW) pixels away from it
        const uint32_t a_tile = desc_lo_kmajor(smem_base + as * p.a_stage_bytes + kRowLead) + (uint32_t)((col - p.PW) * 8);
        if (p.resident) {
          const uint32_t b_cc = b_lo0 + (uint32_t)(cc * taps) * tap_step;
          if (elect_one()) {
            if (FK == 3) {
#pragma unroll
              for (int kh = 0; kh < 3; ++kh)
#pragma unroll
                for (int kw = 0; kw < 3; ++kw)
#pragma unroll
                  for (int k = 0; k < 4; ++k)
#pragma unroll
                    for (int m = 0; m < MT; ++m)
                      mma_tf32_words(d_tmem + m * BN, a_tile + m * tile_step + kh * row_step + kw * 8 + 2 * k, a_hi,
                                     b_cc + (kh * 3 + kw) * tap_step + k * b_step, b_hi, idesc, (kh + kw + k) ? 1u : (uint32_t)(cc > 0));
            } else {
              uint32_t a_row = a_tile, a_lo = a_tile, b_lo = b_cc;
              int kw = 0;
              for (int tap = 0; tap < taps; ++tap, b_lo += tap_step) {
#pragma unroll
                for (int k = 0; k < 4; ++k)
#pragma unroll
                  for (int m = 0; m < MT; ++m)
                    mma_tf32_words(d_tmem + m * BN, a_lo + m * tile_step + 2 * k, a_hi, b_lo + k * b_step, b_hi, idesc, (tap + k) ? 1u : (uint32_t)(cc > 0));
                a_lo += 8u;
                if (++kw == p.KW) { kw = 0; a_row += row_step; a_lo = a_row; }
              }
            }
            mma_commit(smem_u32(&bar_aempty[as]));
          }
          __syncwarp();
        } else if (FK == 3) {
          // streamed weights, 3x3 filter: one filter row (3 taps) per weight stage, straight-line issue
#pragma unroll
          for (int kh = 0; kh < 3; ++kh) {
            ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_bfull[bs]), (uint32_t)blap & 1u, abort_ptr, 15));
            if (!ok) break;
            if (kh == 2 && cc == p.cchunks - 1) *(volatile int*)&tiles_seen = t + 1;
            tc_fence_after();
            const uint32_t b_row = b_lo0 + bs * (b_stage_bytes >> 4);
            if (elect_one()) {
#pragma unroll
              for (int kw = 0; kw < 3; ++kw)
#pragma unroll
                for (int k = 0; k < 4; ++k)
#pragma unroll
                  for (int m = 0; m < MT; ++m)
                    mma_tf32_words(d_tmem + m * BN, a_tile + m * tile_step + kh * row_step + kw * 8 + 2 * k, a_hi, b_row + kw * tap_step + k * b_step,
                                   b_hi, idesc, (kh + kw + k) ? 1u : (uint32_t)(cc > 0));
              mma_commit(smem_u32(&bar_bempty[bs]));
            }
            __syncwarp();
            if (++bs == BST) { bs = 0; ++blap; }
          }
          if (ok && elect_one()) mma_commit(smem_u32(&bar_aempty[as]));
          __syncwarp();
        } else {
          int kh = 0, kw = 0;
          for (int tap0 = 0; tap0 < taps && ok; tap0 += p.tps) {
            const int cnt = taps - tap0 < p.tps ? taps - tap0 : p.tps;
            ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_bfull[bs]), (uint32_t)blap & 1u, abort_ptr, 15));
            if (!ok) break;
            if (tap0 + p.tps >= taps && cc == p.cchunks - 1) *(volatile int*)&tiles_seen = t + 1;
            tc_fence_after();
            if (elect_one()) {
              uint32_t b_lo = b_lo0 + bs * (b_stage_bytes >> 4);
              uint32_t a_lo = a_tile + kh * row_step + kw * 8;
              int w = kw;
              for (int j = 0; j < cnt; ++j, b_lo += tap_step) {
#pragma unroll
                for (int k = 0; k < 4; ++k)
#pragma unroll
                  for (int m = 0; m < MT; ++m)
                    mma_tf32_words(d_tmem + m * BN, a_lo + m * tile_step + 2 * k, a_hi, b_lo + k * b_step, b_hi, idesc,
                                   (tap0 + j + k) ? 1u : (uint32_t)(cc > 0));
                a_lo += 8u;
                if (++w == p.KW) { w = 0; a_lo += row_step - (uint32_t)p.KW * 8u; }
              }
              mma_commit(smem_u32(&bar_bempty[bs]));
            }
            __syncwarp();
            kw += cnt;
            while (kw >= p.KW) { kw -= p.KW; ++kh; }
            if (++bs == BST) { bs = 0; ++blap; }
          }
          if (ok && elect_one()) mma_commit(smem_u32(&bar_aempty[as]));
          __syncwarp();
        }
        if (++as == kRowAStages) { as = 0; ++alap; }
      }
      if (ok && elect_one()) mma_commit(smem_u32(&bar_tfull[buf]));
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------ epilogue (the last four warps)
    const int quarter = warp & 3;
    int t = 0;
    const bool vec_ok = (p.ldo % 4 == 0) &&
                        (((reinterpret_cast<uintptr_t>(p.out) | reinterpret_cast<uintptr_t>(p.bias) | reinterpret_cast<uintptr_t>(p.addend)) & 15u) == 0);
    const bool wide_ok = vec_ok && (p.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 31u) == 0);  // 32-byte stores
    // statistics variant: narrow tiles keep per-lane sums (cheap per tile), wide tiles merge per tile
    constexpr bool LANE_SUMS = STATS && BN == 64;
    WarpColStats<(STATS && !LANE_SUMS) ? BN / 32 : 1> stats;
    LaneColSums<LANE_SUMS ? BN / 32 : 1> sums;
    if constexpr (LANE_SUMS) sums.reset(); else stats.reset();
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++t) {
      const int q_item = (tile / p.n_tiles) * (128 * MT) + quarter * 32 + lane;
      const int n0 = (tile % p.n_tiles) * BN;
      const int buf = t & 1;
      const uint32_t use = (uint32_t)(t >> 1);
      // position -> pixel; padding columns and separator rows have no output
      long long ooff[MT];
      bool valid[MT];
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const int q = q_item + 128 * m;
        const int v = q / p.Wp;
        const int wp = q - v * p.Wp;
        const int img = v / p.Hv;
        const int hrow = v - img * p.Hv;
        valid[m] = q < p.Q && hrow < p.H && wp >= p.PW && wp < p.W + p.PW;
        ooff[m] = (((long long)img * p.H + hrow) * p.W + (wp - p.PW)) * p.ldo;
      }
      // With one tile per item the addend row is fetched while the MMAs of this tile still run:
      // loading it after the accumulator is ready would put a memory round trip per 32 columns
      // into the epilogue, which then takes longer than the main loop of a tile.
      constexpr int kPre = (MT == 1 && BN <= 128) ? BN / 4 : 1;
      float4 pre[kPre];
      const bool prefetched = MT == 1 && BN <= 128 && p.addend != nullptr && valid[0] && vec_ok && n0 + BN <= p.N;
      if (prefetched) {
#pragma unroll
        for (int j = 0; j < kPre; ++j) pre[j] = __ldg(reinterpret_cast<const float4*>(p.addend + ooff[0] + n0) + j);
      }
      bool ok = lane != 0 || mbar_wait(smem_u32(&bar_tfull[buf]), use & 1u, abort_ptr, 16);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if constexpr (BN == 64 && MT == 1) {
        // Narrow tiles, whole column tile, 32-byte aligned rows: every lane stores runs of eight floats (whole
        // sectors).  With statistics the accumulator is read out whole and handed back to the issuing warps
        // before the arithmetic; without, reading and storing half by half measured faster.
        if (wide_ok && n0 + 64 <= p.N && !p.addend) {
          const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN);
          float* orow = p.out + ooff[0] + n0;
          auto put = [&](const uint32_t (&r)[32], int c0) {
            if (!valid[0]) return;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              float o[8];
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                o[k] = __uint_as_float(r[j + k]) + (p.bias ? __ldg(p.bias + n0 + c0 + j + k) : 0.f);
                if (p.relu) o[k] = fmaxf(o[k], 0.f);
              }
              st_global_v8(orow + c0 + j, o[0], o[1], o[2], o[3], o[4], o[5], o[6], o[7]);
            }
          };
          if constexpr (STATS) {
            uint32_t r0[32], r1[32];
            tmem_ld_32x32(t_addr, r0);
            tmem_ld_32x32(t_addr + 32, r1);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[buf]));
            put(r0, 0);
            put(r1, 32);
            // per-lane sums of the raw accumulator (the bias is the pivot)
            if (valid[0]) { sums.add_chunk(0, r0); sums.add_chunk(1, r1); }
            sums.cnt += valid[0] ? 1.f : 0.f;
          } else {
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 32) {
              uint32_t r[32];
              tmem_ld_32x32(t_addr + c0, r);
              tmem_ld_wait();
              put(r, c0);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[buf]));
          }
          continue;
        }
      }
      if constexpr (STATS) {
        // forward convolution feeding a BatchNorm layer (no addend, N % 32 == 0, aligned: checked on the
        // host): store the rows and fold them into the per-channel statistics
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          float* orow = p.out + ooff[m];
          const float cnt = (float)__popc(__ballot_sync(0xffffffffu, valid[m]));
#pragma unroll
          for (int c0 = 0; c0 < BN; c0 += 32) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)((buf * MT + m) * BN + c0), r);
            tmem_ld_wait();
            const int col0 = n0 + c0;
            if (col0 < p.N) {  // warp-uniform
              float o[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) o[j] = __uint_as_float(r[j]) + (p.bias ? __ldg(p.bias + col0 + j) : 0.f);
              if (valid[m]) {
#pragma unroll
                for (int j = 0; j < 32; j += 8)
                  st_row8(orow + col0 + j, make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]), make_float4(o[j + 4], o[j + 5], o[j + 6], o[j + 7]), wide_ok);
              }
              if constexpr (LANE_SUMS) {
                if (valid[m]) sums.add_chunk(c0 / 32, r);
              } else {
                if (cnt > 0.f) stats.add_chunk(c0 / 32, o, valid[m], cnt, lane);
              }
            }
          }
          if constexpr (LANE_SUMS) sums.cnt += valid[m] ? 1.f : 0.f; else stats.n += cnt;
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[buf]));
        continue;
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        float* orow = p.out + ooff[m];
        const float* arow = p.addend ? p.addend + ooff[m] : nullptr;
#pragma unroll
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)((buf * MT + m) * BN + c0), r);
          tmem_ld_wait();
          const int col0 = n0 + c0;
          if (valid[m] && col0 < p.N) {
            if (vec_ok && col0 + 32 <= p.N) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                float4 o[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                  const int jj = j + 4 * h;
                  o[h] = make_float4(__uint_as_float(r[jj]), __uint_as_float(r[jj + 1]), __uint_as_float(r[jj + 2]), __uint_as_float(r[jj + 3]));
                  if (p.bias) {
                    const float4 b = *reinterpret_cast<const float4*>(p.bias + col0 + jj);
                    o[h].x += b.x; o[h].y += b.y; o[h].z += b.z; o[h].w += b.w;
                  }
                  if (arow) {
                    const float4 b = prefetched ? pre[kPre > 1 ? (c0 + jj) / 4 : 0] : *reinterpret_cast<const float4*>(arow + col0 + jj);
                    o[h].x += b.x; o[h].y += b.y; o[h].z += b.z; o[h].w += b.w;
                  }
                  if (p.relu) { o[h].x = fmaxf(o[h].x, 0.f); o[h].y = fmaxf(o[h].y, 0.f); o[h].z = fmaxf(o[h].z, 0.f); o[h].w = fmaxf(o[h].w, 0.f); }
                }
                st_row8(orow + col0 + j, o[0], o[1], wide_ok);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (col0 + j < p.N) {
                  float o = __uint_as_float(r[j]);
                  if (p.bias) o += p.bias[col0 + j];
                  if (arow) o += arow[col0 + j];
                  if (p.relu) o = fmaxf(o, 0.f);
                  orow[col0 + j] = o;
                }
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[buf]));
    }
    if constexpr (STATS) {
      float* row = p.stats + ((long long)(blockIdx.x / p.n_tiles) * 4 + quarter) * 3 * p.N;
      if constexpr (LANE_SUMS) sums.store(row, p.N, (blockIdx.x % p.n_tiles) * BN, p.N, p.bias, lane);
      else stats.store(row, p.N, (blockIdx.x % p.n_tiles) * BN, p.N, lane);
    }
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);  // let copies in flight land before shared memory is released
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * MT * BN);
  }
}

// Geometry and shared-memory plan; `ok` is false when the shape is outside what the kernel
// handles or when too much of the work would land on padding.
struct RowConvPlan {
  bool ok;
  int Wp, Hv, nr_max, b_stages, tps, resident, mt;
  uint32_t a_stage_bytes, smem_bytes;
};

// One candidate layout: mt tiles per work item.
static bool row_conv_layout(RowConvPlan& r, int mt, int ph, int pw, int taps, int kc, int nout, int bn, bool allow_resident) {
  r.mt = mt;
  r.nr_max = (r.Wp - 1 + 128 * mt - 1) / r.Wp + 1 + 2 * ph;
  const uint32_t need = kRowLead + (uint32_t)(r.nr_max * r.Wp + pw + 8) * 128u;
  r.a_stage_bytes = (need + 1023u) & ~1023u;
  const uint32_t budget = 227u * 1024u - 2048u;
  const uint32_t fixed = 1024u + kRowAStages * r.a_stage_bytes;
  const uint32_t tap_bytes = (uint32_t)bn * 128u;
  if (fixed + 3u * tap_bytes > budget) return false;
  const uint32_t filter_bytes = (uint32_t)taps * (kc / 32) * tap_bytes;
  r.resident = 0;
  if (allow_resident && nout <= bn && fixed + filter_bytes <= budget) {  // the whole filter fits beside the activation ring
    r.resident = 1;
    r.tps = taps;
    r.b_stages = 1;
    r.smem_bytes = fixed + filter_bytes;
    return true;
  }
  // the most taps per weight stage that still leaves two stages (hand-overs are expensive)
  int tps = (int)((budget - fixed) / (2u * tap_bytes));
  if (tps > taps) tps = taps;
  if (bn >= 256 || tps < 2) tps = 1;  // N = 256: four MMAs already outlast a hand-over
  if (taps == 9 && tps >= 3) tps = 3;  // 3x3: one filter row per stage, which the unrolled issue path expects
  r.tps = tps;
  int bst = (int)((budget - fixed) / (tps * tap_bytes));
  r.b_stages = bst > 8 ? 8 : bst;
  r.smem_bytes = fixed + r.b_stages * tps * tap_bytes;
  return true;
}

RowConvPlan row_conv_plan(int n, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int kc, int nout, int bn) {
  RowConvPlan r{};
  if (getenv("MTB_DISABLE_ROWCONV")) return r;
  if (sh != 1 || sw != 1 || kh != 2 * ph + 1 || kw != 2 * pw + 1 || kh * kw < 2 || kh * kw > 64 || pw > 7 || kc % 32) return r;
  r.Wp = w + 2 * pw;
  r.Hv = h + ph;
  if (r.Wp > 256) return r;
  if ((double)w * h < 0.8 * (double)r.Wp * r.Hv) return r;  // too much padding: the im2col kernel wastes nothing
  if ((long long)n * r.Hv * r.Wp > 0x7ffff000LL) return r;   // the kernel indexes positions with 32-bit integers
  const int taps = kh * kw;
  if (!row_conv_layout(r, 1, ph, pw, taps, kc, nout, bn, true)) return r;
  r.ok = true;
  // Streamed weights: let two tiles share every weight stage when that still fills the GPU.
  if (!r.resident && bn <= 128 && !getenv("MTB_ROWCONV_MT1")) {
    const long long items = (((long long)n * r.Hv * r.Wp + 255) / 256) * ((nout + bn - 1) / bn);
    RowConvPlan r2 = r;
    const long long min_items = getenv("MTB_ROWCONV_MIN_ITEMS") ? atoll(getenv("MTB_ROWCONV_MIN_ITEMS")) : 2LL * mtb_sm_count();
    if (items >= min_items && row_conv_layout(r2, 2, ph, pw, taps, kc, nout, bn, false) && r2.tps >= 2) r = r2;
  }
  return r;
}

template <int BN, int BMODE, int FK, int MT, bool STATS>
int launch_row_conv_kernel(const CUtensorMap& mapA, const CUtensorMap& mapB, const RowConvParams& p, uint32_t smem_bytes, cudaStream_t st) {
  auto kernel = tc_conv_rows_kernel<BN, BMODE, FK, MT, STATS>;
  static unsigned long long configured = 0;
  if (int rc = mtb_opt_in_smem((const void*)kernel, 227 * 1024 - 1024, &configured)) return rc;
  const int items = ((p.m_tiles + MT - 1) / MT) * p.n_tiles;
  int grid = items < mtb_sm_count() ? items : mtb_sm_count();
  if (STATS) grid = grid / p.n_tiles * p.n_tiles;  // every CTA stays on one output-channel tile
  kernel<<<grid, kRowThreads, smem_bytes, st>>>(mapA, mapB, p);
  MTB_LAUNCH_CHECK("tc_conv_rows_kernel");
  return MTB_OK;
}

// the statistics variant exists for the forward role only (K-major weights)
template <int BN, int BMODE, int FK, int MT>
int launch_row_conv(const CUtensorMap& mapA, const CUtensorMap& mapB, const RowConvParams& p, uint32_t smem_bytes, cudaStream_t st) {
  if constexpr (BMODE == B_KMAJOR) {
    if (p.stats) return launch_row_conv_kernel<BN, BMODE, FK, MT, true>(mapA, mapB, p, smem_bytes, st);
  }
  return launch_row_conv_kernel<BN, BMODE, FK, MT, false>(mapA, mapB, p, smem_bytes, st);
}

// Partial-statistics rows the STATS variant writes (see RowConvParams::stats).
int row_conv_stats_rows(const RowConvPlan& plan, long long positions, int nout, int bn);

template <int BMODE>
int launch_row_conv_bn(int bn, int mt, const CUtensorMap& mapA, const CUtensorMap& mapB, const RowConvParams& p, uint32_t smem_bytes, cudaStream_t st) {
  // the 3x3 filter has its MMA sequence unrolled (weights resident, or streamed one filter row per stage)
  const bool k3 = p.KH == 3 && p.KW == 3 && (p.resident || p.tps == 3);
  if (mt == 2) {  // streamed weights only, BN <= 128
    if (bn == 64) return k3 ? launch_row_conv<64, BMODE, 3, 2>(mapA, mapB, p, smem_bytes, st) : launch_row_conv<64, BMODE, 0, 2>(mapA, mapB, p, smem_bytes, st);
    return k3 ? launch_row_conv<128, BMODE, 3, 2>(mapA, mapB, p, smem_bytes, st) : launch_row_conv<128, BMODE, 0, 2>(mapA, mapB, p, smem_bytes, st);
  }
  if (bn == 64) return k3 ? launch_row_conv<64, BMODE, 3, 1>(mapA, mapB, p, smem_bytes, st) : launch_row_conv<64, BMODE, 0, 1>(mapA, mapB, p, smem_bytes, st);
  if (bn == 128) return k3 ? launch_row_conv<128, BMODE, 3, 1>(mapA, mapB, p, smem_bytes, st) : launch_row_conv<128, BMODE, 0, 1>(mapA, mapB, p, smem_bytes, st);
  return k3 ? launch_row_conv<256, BMODE, 3, 1>(mapA, mapB, p, smem_bytes, st) : launch_row_conv<256, BMODE, 0, 1>(mapA, mapB, p, smem_bytes, st);
}

// Shared by forward (x, K-major weights) and the stride-1 data gradient (dY, weights in place).
// act: [N, H, W, kc] channels-last; out: [N, H, W, nout].
template <int BMODE>
int run_row_conv(const RowConvPlan& plan, int bn, int n, int h, int w, int kc, int kh, int kw, int ph, int pw, int nout, const float* act,
                 const CUtensorMap& mapB, const int* b_tap_x, const float* bias, const float* addend, int relu, float* out, cudaStream_t st,
                 float* stats = nullptr) {
  CUtensorMap mapA;
  int rc = tc::encode_rows_4d(&mapA, act, n, h, w, kc, 32, plan.Wp);
  if (rc) return rc;
  RowConvParams p{};
  p.Q = (long long)n * plan.Hv * plan.Wp;
  p.Wp = plan.Wp; p.Hv = plan.Hv; p.H = h; p.W = w; p.PH = ph; p.PW = pw; p.KH = kh; p.KW = kw;
  p.cchunks = kc / 32; p.kc_total = kc; p.N = nout;
  p.m_tiles = (int)((p.Q + 127) / 128); p.n_tiles = (nout + bn - 1) / bn;
  p.a_stage_bytes = plan.a_stage_bytes; p.b_stages = plan.b_stages; p.tps = plan.tps; p.resident = plan.resident;
  p.out = out; p.ldo = nout; p.bias = bias; p.addend = addend; p.relu = relu;
  p.issuers = getenv("MTB_ROWCONV_ONE_ISSUER") ? 1 : kRowIssuers;
  p.stats = stats;
  if (b_tap_x) for (int j = 0; j < kh * kw; ++j) p.b_tap_x[j] = b_tap_x[j];
  return launch_row_conv_bn<BMODE>(bn, plan.mt, mapA, mapB, p, plan.smem_bytes, st);
}

int row_conv_stats_rows(const RowConvPlan& plan, long long positions, int nout, int bn) {
  const long long m_tiles = (positions + 127) / 128;
  const int n_tiles = (nout + bn - 1) / bn;
  const long long items = ((m_tiles + plan.mt - 1) / plan.mt) * n_tiles;
  const int grid = (int)(items < mtb_sm_count() ? items : mtb_sm_count());
  return grid / n_tiles * 4;
}

}  // namespace

// ------------------------------------------------------------------------------ weight gradient
//
// dW[co][kh][kw][ci] = sum over positions q of dY[q][co] * X[q + (kh-PH)*Wp + (kw-PW)][ci], in the
// same padded linear position space as above (dY is staged with the same zero-filled padding
// columns and separator rows, so padding positions contribute nothing).  Both operands lie in
// shared memory as [position][32 channels] panels, which tcgen05 reads as MN-major operands with
// the position as the reduction index.  A filter tap is a shift of the X panel by whole rows, and
// the four 32-wide M blocks of one MMA are the SAME X panel shifted by 0, 1, 2, 3 positions
// (descriptor LBO = 128 bytes): one MMA covers kw = 0..3 of one filter row for 32 input channels
// (for a 3-wide filter the fourth block is computed and dropped).  X and dY are therefore staged
// once per block of 128 positions instead of once per tap, which is what bounded the im2col
// form (the copy engine pays per 128-byte pixel row it gathers).
//
// One CTA = one unit (group of input-channel blocks, range of position blocks); it keeps one
// accumulator of BN columns per (channel block, filter row, group of 4 taps) in tensor memory and
// writes them as an fp32 partial; the partials are added in a fixed order afterwards.
namespace {

struct WgradRowsParams {
  long long Q;
  int Wp, Hv, H, W, PH, PW, KH, KW;
  int Cin, Cout;
  int ncc_g;     // channel blocks of 32 per group
  int n_tiles;   // output-channel tiles of BN
  int n_kwg;     // ceil(KW / 4)
  int splits, kb_total, kb_per_split;  // position blocks of 128
  uint32_t x_panel_bytes, y_panel_bytes, stage_bytes;
  float* partial;  // [splits][KH*KW*Cin][Cout]
};

constexpr int kWgRowsStages = 2;
constexpr int kWgRowsPB = 128;  // positions per stage

// FIX > 0: 3-tall, at most 4-wide filter with exactly FIX channel blocks per CTA; the MMA sequence of
// a stage is then straight-line code (issuing from runtime loops costs twice the cycles per MMA).
template <int BN, int FIX>
__global__ void __launch_bounds__(192, 1)
tc_wgrad_rows_kernel(const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapDY, const WgradRowsParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_full[kWgRowsStages], bar_empty[kWgRowsStages], bar_tfull;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

  // lead / tail rows of the panels are read (against zero gradients only) but never written
  for (uint32_t i = threadIdx.x; i < kWgRowsStages * p.stage_bytes / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(smem_raw + (smem_base - smem_u32(smem_raw)))[i] = make_uint4(0, 0, 0, 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kWgRowsStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    mbar_init(smem_u32(&bar_tfull), 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), 512);
    tmem_relinquish();
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  volatile int* abort_ptr = &abort_flag;

  const int split = blockIdx.x % p.splits;
  const int n0 = ((blockIdx.x / p.splits) % p.n_tiles) * BN;
  const int group = blockIdx.x / (p.splits * p.n_tiles);
  const int cchunks = p.Cin / 32;
  const int cc0 = group * p.ncc_g;
  const int ncc = cchunks - cc0 < p.ncc_g ? cchunks - cc0 : p.ncc_g;
  const int kb0 = split * p.kb_per_split;
  const int kb1 = kb0 + p.kb_per_split < p.kb_total ? kb0 + p.kb_per_split : p.kb_total;
  const uint32_t row_bytes = (uint32_t)p.Wp * 128u;
  const uint32_t y_off = (uint32_t)p.ncc_g * p.x_panel_bytes;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&mapX);
      prefetch_tensormap(&mapDY);
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        const long long q0 = (long long)kb * kWgRowsPB;
        const int v0 = (int)(q0 / p.Wp);
        const int nr_y = (int)((q0 + kWgRowsPB - 1) / p.Wp) - v0 + 1;
        const int nr_x = nr_y + 2 * p.PH;
        if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abort_ptr, 21)) break;
        const uint32_t full = smem_u32(&bar_full[stage]);
        mbar_expect_tx(full, (uint32_t)(nr_x * ncc + nr_y * (BN / 32)) * row_bytes);
        const uint32_t st = smem_base + stage * p.stage_bytes;
        {
          const int v = v0 - p.PH;
          int im = v >= 0 ? v / p.Hv : -1, hr = v - im * p.Hv;
          uint32_t dst = st + kRowLead;
          for (int r = 0; r < nr_x; ++r, dst += row_bytes) {
            for (int c = 0; c < ncc; ++c) tma_load_4d(dst + c * p.x_panel_bytes, &mapX, full, (cc0 + c) * 32, -p.PW, hr, im);
            if (++hr == p.Hv) { hr = 0; ++im; }
          }
        }
        {
          int im = v0 / p.Hv, hr = v0 - im * p.Hv;
          uint32_t dst = st + y_off;
          for (int r = 0; r < nr_y; ++r, dst += row_bytes) {
#pragma unroll
            for (int j = 0; j < BN / 32; ++j) tma_load_4d(dst + j * p.y_panel_bytes, &mapDY, full, n0 + j * 32, -p.PW, hr, im);
            if (++hr == p.Hv) { hr = 0; ++im; }
          }
        }
        if (++stage == kWgRowsStages) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (converged warp, elected issue)
    constexpr uint32_t idesc = idesc_tf32(128, BN, 1, 1);
    constexpr uint32_t hi = desc_hi_mnmajor();
    const uint32_t wp8 = (uint32_t)p.Wp * 8u;  // one image row in 16-byte units
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int col0 = (int)(((long long)kb0 * kWgRowsPB) % p.Wp);
    for (int kb = kb0; kb < kb1 && ok; ++kb) {
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_full[stage]), phase, abort_ptr, 22));
      if (!ok) break;
      tc_fence_after();
      const uint32_t st = smem_base + stage * p.stage_bytes;
      // position q0 sits PH rows and col0 pixels into the X rows, col0 pixels into the dY rows
      const uint32_t x_lo = desc_lo_mnmajor(st + kRowLead, 128u) + (uint32_t)((col0 - p.PW) * 8);
      const uint32_t y_lo = desc_lo_mnmajor(st + y_off, p.y_panel_bytes) + (uint32_t)(col0 * 8);
      const uint32_t x_panel = p.x_panel_bytes >> 4;
      if (elect_one()) {
        if (FIX > 0) {
          const uint32_t first = kb > kb0 ? 1u : 0u;
#pragma unroll
          for (int ks = 0; ks < kWgRowsPB / 8; ++ks)  // 8 positions per MMA; 8 rows of 128 B = 64 units
#pragma unroll
            for (int c = 0; c < FIX; ++c)
#pragma unroll
              for (int kh = 0; kh < 3; ++kh)
                mma_tf32_words(tmem_base + (c * 3 + kh) * BN, x_lo + c * x_panel + kh * wp8 + ks * 64u, hi, y_lo + ks * 64u, hi, idesc, ks ? 1u : first);
        } else {
          for (int ks = 0; ks < kWgRowsPB / 8; ++ks) {
            const uint32_t accum = (kb > kb0 || ks > 0) ? 1u : 0u;
            const uint32_t yk = y_lo + ks * 64u;
            uint32_t d = tmem_base;
            for (int c = 0; c < ncc; ++c) {
              uint32_t xk = x_lo + c * x_panel + ks * 64u;
              for (int kh = 0; kh < p.KH; ++kh, xk += wp8)
                for (int g = 0; g < p.n_kwg; ++g, d += BN) mma_tf32_words(d, xk + g * 32u, hi, yk, hi, idesc, accum);
            }
          }
        }
        mma_commit(smem_u32(&bar_empty[stage]));
      }
      __syncwarp();
      col0 = (col0 + kWgRowsPB) % p.Wp;
      if (++stage == kWgRowsStages) { stage = 0; phase ^= 1u; }
    }
    if (ok && elect_one()) mma_commit(smem_u32(&bar_tfull));
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;
    bool ok = lane != 0 || mbar_wait(smem_u32(&bar_tfull), 0, abort_ptr, 23);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      const long long Kw = (long long)p.KH * p.KW * p.Cin;
      float* part = p.partial + (long long)split * Kw * p.Cout;
      const bool vec_ok = (p.Cout % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.partial) & 15u) == 0);
      const bool wide_ok = (p.Cout % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.partial) & 31u) == 0);
      int a = 0;
      for (int c = 0; c < ncc; ++c)
        for (int kh = 0; kh < p.KH; ++kh)
          for (int g = 0; g < p.n_kwg; ++g, ++a) {
            const int kw = g * 4 + quarter;             // M block = tap within the group of four
            const int ci = (cc0 + c) * 32 + lane;
            const bool valid = kw < p.KW && ci < p.Cin;
            float* orow = part + ((long long)(kh * p.KW + kw) * p.Cin + ci) * p.Cout + n0;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
              uint32_t r[32];
              tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(a * BN + c0), r);
              tmem_ld_wait();
              if (valid && n0 + c0 < p.Cout) {
                if (vec_ok && n0 + c0 + 32 <= p.Cout) {
#pragma unroll
                  for (int j = 0; j < 32; j += 8)
                    st_row8(orow + c0 + j, make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])),
                            make_float4(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]), __uint_as_float(r[j + 6]), __uint_as_float(r[j + 7])), wide_ok);
                } else {
#pragma unroll
                  for (int j = 0; j < 32; ++j)
                    if (n0 + c0 + j < p.Cout) orow[c0 + j] = __uint_as_float(r[j]);
                }
              }
            }
          }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// dw[co][r] = sum_s partial[s][r][co] with the splits spread over 8 thread groups (group z adds
// splits z, z+8, ... in order; the 8 sums are then added in index order): the same result for
// any launch, and enough CTAs to read ~100 partial planes at full speed.
__global__ void __launch_bounds__(1024) wgrad_reduce_many_kernel(const float* __restrict__ partial, float* __restrict__ dw, int Kw, int Cout, int splits) {
  __shared__ float acc[8][4][33];
  const int c = blockIdx.y * 32 + threadIdx.x;
  const int r = blockIdx.x * 4 + threadIdx.y;
  const int z0 = threadIdx.z;
  const long long plane = (long long)Kw * Cout;
  float s0 = 0.f, s1 = 0.f;
  if (r < Kw && c < Cout) {
    const float* q = partial + (long long)r * Cout + c;
    int z = z0;
    for (; z + 8 < splits; z += 16) { s0 += q[z * plane]; s1 += q[(z + 8) * plane]; }
    if (z < splits) s0 += q[z * plane];
  }
  acc[z0][threadIdx.y][threadIdx.x] = s0 + s1;
  __syncthreads();
  if (z0 == 0 && r < Kw && c < Cout) {
    float t = acc[0][threadIdx.y][threadIdx.x];
#pragma unroll
    for (int k = 1; k < 8; ++k) t += acc[k][threadIdx.y][threadIdx.x];
    dw[(long long)c * Kw + r] = t;
  }
}

struct WgradRowsPlan {
  bool ok;
  int bn, n_tiles, Wp, Hv, ncc_g, groups, n_kwg, splits, kb_total, kb_per_split;
  uint32_t x_panel_bytes, y_panel_bytes, stage_bytes, smem_bytes;
};

WgradRowsPlan wgrad_rows_plan(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout) {
  WgradRowsPlan r{};
  if (getenv("MTB_DISABLE_ROWCONV") || getenv("MTB_DISABLE_ROWWGRAD")) return r;
  if (sh != 1 || sw != 1 || kh != 2 * ph + 1 || kw != 2 * pw + 1 || kh * kw < 2 || pw > 7 || cin % 32 || cout > 256 || cout % 4) return r;
  // 64-wide output tiles: two channel blocks' accumulators fit in tensor memory side by side, so X
  // and dY panels are each staged for 96 MMAs instead of 48
  r.bn = (cout <= 64 || !getenv("MTB_WGRAD_BN128")) ? 64 : 128;
  r.n_tiles = (cout + r.bn - 1) / r.bn;
  r.Wp = w + 2 * pw;
  r.Hv = h + ph;
  r.n_kwg = (kw + 3) / 4;
  if (r.Wp > 256) return r;
  // useful share of the MMA work: padding positions and the unused taps of the last group of four
  if ((double)w * h * kw < 0.6 * (double)r.Wp * r.Hv * (4 * r.n_kwg)) return r;
  const int nr_y = (r.Wp - 1 + kWgRowsPB - 1) / r.Wp + 1, nr_x = nr_y + 2 * ph;
  r.x_panel_bytes = (kRowLead + (uint32_t)(nr_x * r.Wp + 16) * 128u + 1023u) & ~1023u;
  r.y_panel_bytes = ((uint32_t)(nr_y * r.Wp) * 128u + 1023u) & ~1023u;
  const uint32_t budget = 227u * 1024u - 3072u;
  const int cchunks = cin / 32;
  int best = 0;
  for (int g = 1; g <= cchunks; ++g) {
    if (kh * r.n_kwg * g * r.bn > 512) break;
    const uint32_t stage = g * r.x_panel_bytes + (r.bn / 32) * r.y_panel_bytes;
    if (kWgRowsStages * stage > budget) break;
    best = g;
  }
  if (best == 0) return r;
  r.ncc_g = best;
  r.groups = (cchunks + best - 1) / best;
  r.stage_bytes = best * r.x_panel_bytes + (r.bn / 32) * r.y_panel_bytes;
  r.smem_bytes = kWgRowsStages * r.stage_bytes + 1024;
  const long long Q = (long long)n * r.Hv * r.Wp;
  r.kb_total = (int)((Q + kWgRowsPB - 1) / kWgRowsPB);
  int splits = mtb_sm_count() / (r.groups * r.n_tiles);
  if (splits < 1) splits = 1;
  if (splits > r.kb_total) splits = r.kb_total;
  r.kb_per_split = (r.kb_total + splits - 1) / splits;
  r.splits = (r.kb_total + r.kb_per_split - 1) / r.kb_per_split;
  r.ok = true;
  return r;
}

template <int BN, int FIX>
int launch_wgrad_rows(const CUtensorMap& mapX, const CUtensorMap& mapDY, const WgradRowsParams& p, int grid, uint32_t smem_bytes, cudaStream_t st) {
  auto kernel = tc_wgrad_rows_kernel<BN, FIX>;
  static unsigned long long configured = 0;
  if (int rc = mtb_opt_in_smem((const void*)kernel, 227 * 1024 - 1024, &configured)) return rc;
  kernel<<<grid, 192, smem_bytes, st>>>(mapX, mapDY, p);
  MTB_LAUNCH_CHECK("tc_wgrad_rows_kernel");
  return MTB_OK;
}

int run_wgrad_rows(const WgradRowsPlan& q, int n, int cin, int h, int w, int kh, int kw, int ph, int pw, int cout, const float* x, const float* dy,
                   float* dw, float* partial, cudaStream_t st) {
  CUtensorMap mapX, mapDY;
  int rc = tc::encode_rows_4d(&mapX, x, n, h, w, cin, 32, q.Wp, true);
  if (rc) return rc;
  rc = tc::encode_rows_4d(&mapDY, dy, n, h, w, cout, 32, q.Wp, true);
  if (rc) return rc;
  WgradRowsParams p{};
  p.Q = (long long)n * q.Hv * q.Wp;
  p.Wp = q.Wp; p.Hv = q.Hv; p.H = h; p.W = w; p.PH = ph; p.PW = pw; p.KH = kh; p.KW = kw;
  p.Cin = cin; p.Cout = cout; p.ncc_g = q.ncc_g; p.n_tiles = q.n_tiles; p.n_kwg = q.n_kwg;
  p.splits = q.splits; p.kb_total = q.kb_total; p.kb_per_split = q.kb_per_split;
  p.x_panel_bytes = q.x_panel_bytes; p.y_panel_bytes = q.y_panel_bytes; p.stage_bytes = q.stage_bytes;
  p.partial = partial;
  const int grid = q.groups * q.n_tiles * q.splits;
  // straight-line MMA sequence when every CTA has the same, small number of channel blocks
  const int fix = (kh == 3 && q.n_kwg == 1 && (cin / 32) % q.ncc_g == 0 && q.ncc_g <= 2) ? q.ncc_g : 0;
  if (q.bn == 64) {
    rc = fix == 2 ? launch_wgrad_rows<64, 2>(mapX, mapDY, p, grid, q.smem_bytes, st)
       : fix == 1 ? launch_wgrad_rows<64, 1>(mapX, mapDY, p, grid, q.smem_bytes, st)
                  : launch_wgrad_rows<64, 0>(mapX, mapDY, p, grid, q.smem_bytes, st);
  } else {
    rc = fix == 1 ? launch_wgrad_rows<128, 1>(mapX, mapDY, p, grid, q.smem_bytes, st) : launch_wgrad_rows<128, 0>(mapX, mapDY, p, grid, q.smem_bytes, st);
  }
  if (rc) return rc;
  const int Kw = kh * kw * cin;
  dim3 rgrid((unsigned)((Kw + 3) / 4), (unsigned)((cout + 31) / 32));
  wgrad_reduce_many_kernel<<<rgrid, dim3(32, 4, 8), 0, st>>>(partial, dw, Kw, cout, q.splits);
  MTB_LAUNCH_CHECK("wgrad_reduce_many_kernel");
  return MTB_OK;
}

}  // namespace
