// Blackwell (sm_100a) building blocks: mbarriers with bounded waits, TMA tensor-map loads
// (tiled and im2col), tcgen05 MMA / commit / TMEM alloc / TMEM load, shared-memory matrix
// descriptors, and host-side tensor-map encoding through the driver entry point.
//
// Every wait on an mbarrier is bounded: when the limit is reached the waiter raises a CTA-wide
// abort flag (which the other roles poll), records a code in g_tc_status and leaves its loop;
// the kernel then tears down normally (TMEM is freed, the CTA exits).  Nothing traps.
#pragma once
#include "common.cuh"
#include <cuda.h>

// Status words of the tensor-core kernels (0 = fine).  One copy per translation unit that
// includes this header; all tcgen05 kernels live in a single translation unit.
static __device__ int g_tc_status[8];

namespace tc {

constexpr long long kWaitCycles = 4000000000LL;  // ~2 s at 1.9 GHz

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Returns false when the wait was abandoned (limit reached here, or another role aborted).
__device__ __forceinline__ bool mbar_wait_limit(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code, long long limit_cycles) {
  if (mbar_try_wait(bar, parity)) return true;
  long long start = clock64();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - start > limit_cycles) {
        *abort_flag = 1;
        atomicCAS(&g_tc_status[0], 0, code);
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
  return mbar_wait_limit(bar, parity, abort_flag, code, kWaitCycles);
}

// 32-byte store (sm_100): a lane that owns a run of eight floats writes whole sectors
__device__ __forceinline__ void st_global_v8(float* p, float a, float b, float c, float d, float e, float f, float g, float h) {
  asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d), "f"(e), "f"(f), "f"(g), "f"(h)
               : "memory");
}

// eight consecutive floats of a row: one 32-byte store where the row allows it (wide), else two 16-byte ones
__device__ __forceinline__ void st_row8(float* p, float4 a, float4 b, bool wide) {
  if (wide) {
    st_global_v8(p, a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w);
  } else {
    *reinterpret_cast<float4*>(p) = a;
    *reinterpret_cast<float4*>(p + 4) = b;
  }
}

// Bounded wait for a shared-memory counter another warp of the CTA advances (kernels with two MMA-issuing
// warps use it to order their parity waits on ring slots that both consume).
__device__ __forceinline__ bool lap_wait(volatile int* seen, int lap, volatile int* abort_flag, int code) {
  if (*seen >= lap) return true;
  const long long start = clock64();
  for (uint32_t it = 1;; ++it) {
    if (*seen >= lap) return true;
    if ((it & 63u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - start > kWaitCycles) {
        *abort_flag = 1;
        atomicCAS(&g_tc_status[0], 0, code);
        return false;
      }
    }
  }
}

// ---- TMA loads (global -> shared, completion on an mbarrier) ----
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
               : "memory");
}
// tiled mode over a channels-last tensor {C, W, H, N}; coordinates outside the tensor read zeros
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c, int w, int h, int n) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n)
               : "memory");
}
// the same box, only brought into L2 (no shared-memory destination, no completion to wait for)
__device__ __forceinline__ void tma_prefetch_4d(const CUtensorMap* map, int c, int w, int h, int n) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global [%0, {%1, %2, %3, %4}];" ::"l"(map), "r"(c), "r"(w), "r"(h), "r"(n) : "memory");
}
// im2col mode over a channels-last tensor {C, W, H, N}: c/w/h/n locate the first pixel (in
// input coordinates, i.e. already multiplied by the stride and shifted by -padding); off_w/off_h
// are the filter-tap offsets.
__device__ __forceinline__ void tma_load_im2col_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c, int w, int h, int n,
                                                   uint16_t off_w, uint16_t off_h) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h)
      : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// One lane of a converged warp (the others skip the guarded block); the warp stays converged, so
// values computed before the block from warp-uniform inputs can live in uniform registers.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}\n" : "=r"(pred));
  return pred != 0;
}

// ---- tcgen05 ----
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem], TF32 inputs, FP32 accumulate; issued by one thread.
__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier receives one arrival when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 columns of 32-bit: thread i of the warp receives columns [col, col+32) of lane
// (lane_base + i).  A warp may only touch the TMEM lane quarter (warp_id % 4).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptors.
// K-major operand (SWIZZLE_128B, TMA swizzle 128B): rows of 128 B hold 32 fp32 of K for one
// M/N index; 16-byte chunks are XOR-swizzled by (row % 8); 8-row groups are `sbo` bytes apart
// (1024 when packed); lbo is unused (encoded as 16 B).
__device__ __forceinline__ uint64_t smem_desc_kmajor(uint32_t saddr, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFFu);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version for sm_100
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}
// MN-major operand of a 32-bit type (the only layout tcgen05 accepts for it: 128-byte swizzle
// with a 32-byte atom base; TMA swizzle 128B_ATOM_32B): rows of 128 B hold 32 consecutive M/N
// elements for one k; 32-byte chunks are XOR-swizzled by (row % 4); 4 rows form one K group;
// `lbo` = bytes between 32-wide M/N blocks, `sbo` = bytes between K groups (512 when packed).
__device__ __forceinline__ uint64_t smem_desc_mnmajor(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFFu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)1 << 61;  // SWIZZLE_128B_BASE32B
  return d;
}

// The same descriptors as two 32-bit words, so that the issuing thread only has to add a small
// constant to the low word per MMA (start address lives in bits 0-13 of the low word).
__host__ __device__ constexpr uint32_t desc_hi_kmajor() { return (1024u >> 4) | (1u << 14) | (2u << 29); }
__host__ __device__ constexpr uint32_t desc_hi_mnmajor() { return (512u >> 4) | (1u << 14) | (1u << 29); }
__device__ __forceinline__ uint32_t desc_lo_kmajor(uint32_t saddr) { return ((saddr >> 4) & 0x3FFFu) | (1u << 16); }
__device__ __forceinline__ uint32_t desc_lo_mnmajor(uint32_t saddr, uint32_t lbo_bytes = 4096u) {
  return ((saddr >> 4) & 0x3FFFu) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}

__device__ __forceinline__ void mma_tf32_words(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 da, db;\n"
      "setp.ne.b32 p, %6, 0;\n"
      "mov.b64 da, {%1, %2};\n"
      "mov.b64 db, {%3, %4};\n"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %5, p;\n"
      "}\n"
      ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate));
}

// Instruction descriptor for kind::tf32, FP32 accumulate, dense, M x N tile.
__host__ __device__ constexpr uint32_t idesc_tf32(int m, int n, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}

// ---- per-channel statistics of the rows an epilogue warp holds ----
//
// An epilogue warp owns 32 output rows (one per lane) and walks the tile's columns in chunks of 32:
// lane i holds v[0..31] = row i, columns c0..c0+31.  warp_transpose_sum adds the 32 lanes' arrays
// column-wise and leaves the sum of column j in lane j (five exchange steps: a lane keeps one half of
// its array and receives the partner's sums for that half).  The array is consumed.
__device__ __forceinline__ float warp_transpose_sum(float (&v)[32], int lane) {
#pragma unroll
  for (int half = 16; half >= 1; half >>= 1) {
    const bool upper = (lane & half) != 0;
#pragma unroll
    for (int k = 0; k < half; ++k) {
      const float keep = upper ? v[k + half] : v[k];
      const float send = upper ? v[k] : v[k + half];
      v[k] = keep + __shfl_xor_sync(0xffffffffu, send, half);
    }
  }
  return v[0];
}

// Running (count, mean, M2) of CHUNKS x 32 columns over all rows a warp has seen; lane j owns column
// j of every chunk.  A tile contributes its mean and centred sum of squares (two column sums over the
// warp's valid rows), merged with Chan's update, so nothing is lost to cancellation when the mean is
// large against the spread.  The convolution epilogues use it to hand BatchNorm its batch statistics
// without a second pass over the output.
template <int CHUNKS>
struct WarpColStats {
  float n, mean[CHUNKS], m2[CHUNKS];
  __device__ __forceinline__ void reset() {
    n = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) { mean[c] = 0.f; m2[c] = 0.f; }
  }
  // o: this lane's row, 32 columns of chunk `c` (compile-time after unrolling); cnt = valid rows in the warp
  __device__ __forceinline__ void add_chunk(int c, const float (&o)[32], bool valid, float cnt, int lane) {
    float t[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) t[k] = valid ? o[k] : 0.f;
    const float mt = warp_transpose_sum(t, lane) / cnt;
#pragma unroll
    for (int k = 0; k < 32; ++k) {
      const float d = o[k] - __shfl_sync(0xffffffffu, mt, k);
      t[k] = valid ? d * d : 0.f;
    }
    const float q = warp_transpose_sum(t, lane);
    const float wb = cnt / (n + cnt);
    const float d = mt - mean[c];
    mean[c] += d * wb;
    m2[c] += q + d * d * n * wb;
  }
  // one partial row [3][C] (count, mean, M2) at columns col0 + 32 c + lane
  __device__ __forceinline__ void store(float* row, int C, int col0, int ncols, int lane) const {
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = col0 + 32 * c + lane;
      if (col < ncols) { row[col] = n; row[C + col] = mean[c]; row[2 * C + col] = m2[c]; }
    }
  }
};

// The cheap form for narrow tiles (64 columns), whose main loop per tile is short enough that every
// instruction an epilogue warp issues is felt by the MMA-issuing warp on the same scheduler: each lane
// keeps plain sums and sums of squares of ITS rows, column by column, in registers (two FADD/FFMA per
// element, no exchange), and the 32 lanes are combined once, when the CTA has finished its tiles.  The
// sums are taken of the raw accumulator, i.e. of y - bias: the bias is the natural pivot of a
// convolution's output, so the single-pass variance loses accuracy only as (mean - bias)^2 / var grows
// (relative error about 6e-8 * (1 + that ratio) * sqrt(rows per lane)).
template <int CHUNKS>
struct LaneColSums {
  float cnt, s1[CHUNKS][32], s2[CHUNKS][32];
  __device__ __forceinline__ void reset() {
    cnt = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
      for (int k = 0; k < 32; ++k) { s1[c][k] = 0.f; s2[c][k] = 0.f; }
  }
  __device__ __forceinline__ void add_chunk(int c, const uint32_t (&r)[32]) {  // raw accumulator row of a valid pixel
#pragma unroll
    for (int k = 0; k < 32; ++k) {
      const float v = __uint_as_float(r[k]);
      s1[c][k] += v;
      s2[c][k] = fmaf(v, v, s2[c][k]);
    }
  }
  // one partial row [3][C] (count, mean, M2); bias (may be NULL) is added back to the mean
  __device__ __forceinline__ void store(float* row, int C, int col0, int ncols, const float* bias, int lane) {
    float n = cnt;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) n += __shfl_xor_sync(0xffffffffu, n, off);
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const float t1 = warp_transpose_sum(s1[c], lane), t2 = warp_transpose_sum(s2[c], lane);
      const int col = col0 + 32 * c + lane;
      if (col < ncols) {
        const float mu = n > 0.f ? t1 / n : 0.f;
        row[col] = n;
        row[C + col] = mu + (bias ? bias[col] : 0.f);
        row[2 * C + col] = n > 0.f ? fmaxf(t2 - t1 * mu, 0.f) : 0.f;
      }
    }
  }
};

// ---- host: tensor maps ----
// fp32 matrix [rows][cols] row-major (row pitch `pitch_elems`), boxes of box_cols x box_rows
// elements, 128-byte swizzle, zero fill outside the matrix.
// mn_major selects the 32-byte-atom swizzle that MN-major tcgen05 operands need.
int encode_tiled_2d(CUtensorMap* map, const float* base, long long rows, long long cols, long long pitch_elems, int box_cols, int box_rows,
                    bool mn_major = false);
// channels-last activation {C, W, H, N}; a load takes `box_w` consecutive pixels of one image
// row x `channels` channels (tiled mode, 128-byte swizzle, zero fill outside the tensor).
int encode_rows_4d(CUtensorMap* map, const float* base, int n, int h, int w, int c, int channels, int box_w, bool mn_major = false);
// channels-last activation {C, W, H, N}; a load takes `pixels` output pixels x `channels`
// channels for one filter tap of a convolution with the given stride / lower padding; `upper`
// = lower_pad - (filter - 1) per spatial dim bounds the walk of the window origin.
int encode_im2col_4d(CUtensorMap* map, const float* base, int n, int h, int w, int c, int lower_w, int lower_h, int upper_w, int upper_h,
                     int stride_w, int stride_h, int channels, int pixels, bool mn_major = false);

}  // namespace tc
