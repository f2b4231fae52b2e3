// TAGI Linear on the 5th-generation tensor cores (tcgen05, sm_100a) with 3xTF32 splitting.
//
// Every FP32 product x*y of the three Linear contractions is evaluated as
//     hi(x)*hi(y) + hi(x)*lo(y) + lo(x)*hi(y),   hi(x) = x with the low 13 mantissa bits cleared,
//                                                 lo(x) = x - hi(x)  (exact in FP32)
// by three kind::tf32 MMAs that accumulate in FP32 in tensor memory. The tensor core reads the
// upper 19 bits of each 32-bit operand, so the raw FP32 tile that TMA lands in shared memory
// already is the hi operand of the B side; the lo tiles and the derived tiles (mu^2 + var, mu^2, and their
// lo parts) are produced by a group of converter warps: B-side tiles elementwise at the same swizzled
// shared-memory offsets as the raw tiles, A-side tiles straight into tensor memory. Nothing derived is ever
// written to HBM.
//
// Two kernels: one CTA per 128 x bn tile of both outputs ("ts", passes with fewer than 256 output rows) and CTA
// pairs on 256 x bn tiles ("pair", everything else). Roles of a CTA's warps:
//   warp 0        TMA producer: raw operand tiles, K-slab of 16, multi-stage ring
//   warps 1, 10   MMA issuers (one thread each): D1 and D2; warp 1 owns tensor memory
//   warps 2-9     converters; they also add finished chunks (tcgen05.ld) to register sums and run the epilogue
//                 (bias / scale -> HBM)
// Operands whose contraction index is contiguous in memory are staged K-major (64-byte swizzle);
// the others (mu_w in the state pass, both operands of the parameter pass) are staged MN-major
// (128-byte swizzle), which kind::tf32 accepts, so no transpose pass exists anywhere.
//
// The tensor core's FP32 accumulation loses a little on every MMA (its error grows with the number of
// MMAs chained into one accumulator and with the accumulator's magnitude), which over thousands of k
// steps would exceed the 1e-5 / 1e-4 tolerance. The contraction is therefore cut into chunks of 256:
// each chunk accumulates from zero in tensor memory and the converter warps add the finished chunk to
// running sums that they keep in registers (plain FP32 adds, one per chunk).
#include <cuda.h>

#include <mutex>

#include "tagi_common.h"

#include <atomic>
#include "tagi_tc_ptx.cuh"
#include "tagi_tc_tile.cuh"

namespace tagi {
namespace {

using namespace ptx;

// K-major tile [128 rows][16 k], 64-byte swizzle: one box. MN-major tile: four boxes of [16 k][32 rows], 2 KiB
// apart, in the 128-byte swizzle with 32-byte atoms, which is the only MN-major layout kind::tf32 reads
// (swizzle pattern repeats every 4 k rows = 512 bytes).
template <int MN>
__device__ __forceinline__ void load_tile(uint32_t dst, const CUtensorMap *tm, int row0, int k0, uint64_t *bar) {
    if (MN) {
#pragma unroll
        for (int g = 0; g < 4; g++) tma_load_2d(dst + g * 2048, tm, row0 + 32 * g, k0, bar);
    } else {
        tma_load_2d(dst, tm, k0, row0, bar);
    }
}

// =====================================================================================================
// Kernel "ts": one CTA per tile, the A-side operand tiles live in tensor memory instead of shared memory.
//
// With every operand tile in shared memory the kernel is bound by shared-memory bandwidth (measured: per k-slab the
// tensor core reads 18 x 8 KiB of operands while the converters read 32 KiB and write 64 KiB). Here the converters write
// the six (forward) or four (backward) A-side tiles straight into tensor memory with tcgen05.st (lane = row, one tf32
// per column) and the MMAs take A from there, which halves the tensor core's shared-memory reads and removes
// the A-side converter writes. Raw tiles and derived B tiles use separate rings so that TMA can run four
// slabs ahead. Tensor memory: columns [0,256) = D1, D2 (one accumulator set; the MMA warp pauses while a
// finished 256-wide contraction chunk is added to the register sums), [256, 256 + 2 x 16 x NA) = A tiles.
// =====================================================================================================
template <int OP> struct TsTraits;
// raw ring slot: A0 A1 B0 B1 (forward) / A0 A1 W (backward); derived slot: B0l B1l Q Ql / Wl Q Ql
template <> struct TsTraits<OP_FWD> { static constexpr int NRAW = 4, NDER = 4, NA = 6; };
template <> struct TsTraits<OP_BWD_STATE> { static constexpr int NRAW = 3, NDER = 3, NA = 4; };
template <> struct TsTraits<OP_BWD_PARAM> { static constexpr int NRAW = 3, NDER = 3, NA = 4; };

// RS raw-ring slots, DS derived-ring slots (shared memory for B, tensor memory for A)
template <int OP, int RS, int DS>
constexpr size_t ts_smem_bytes() {
    return at_least_stage((size_t)(RS * TsTraits<OP>::NRAW + DS * TsTraits<OP>::NDER) * TILE_BYTES) + 1024 + 256;
}

template <int OP, int CH, int RS, int DS>
// 11 warps: three share one SM sub-partition (16 K registers), which caps a thread at 168 registers
__global__ void __launch_bounds__(NTHREADS2, 1)
tagi_tc_linear_ts_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
                         const __grid_constant__ CUtensorMap tmB0, const __grid_constant__ CUtensorMap tmB1,
                         const TcEpilogue epi, const int kdim, const int bn, int *status) {
    using T = OpTraits<OP>;
    using S = TsTraits<OP>;
    constexpr int NRAW = S::NRAW, NDER = S::NDER, NA = S::NA;
    constexpr uint32_t NCOLS = 512;
    // tensor-memory columns: D1 at 0, D2 at acc_stride, A tiles from 2 * acc_stride on (DS slots of NA * 16 columns)
    const uint32_t acc_stride = (512 - DS * NA * BK) / 2 >= 128 ? 128 : 112;
    const uint32_t A_COL0 = 2 * acc_stride;
    const uint32_t IDESC = make_idesc_tf32(TM, bn, 0, T::B_MN);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *aligned = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t raw_base = smem_base, der_base = smem_base + RS * NRAW * TILE_BYTES;
    // the epilogue stages its tile over the rings, so the barriers sit behind whichever is larger
    uint64_t *bars = reinterpret_cast<uint64_t *>(aligned + at_least_stage((size_t)(RS * NRAW + DS * NDER) * TILE_BYTES));
    // stage_done[it % L] completes when the MMAs of k-slab `it` have finished: one commit per slab releases both the
    // raw slot (refilled RS slabs later) and the derived slot (overwritten DS slabs later)
    constexpr int L = RS > DS ? RS : DS;
    uint64_t *raw_full = bars, *stage_done = bars + RS, *conv_done = bars + RS + L;
    uint64_t *acc_full = bars + RS + L + DS, *acc_empty = acc_full + 1;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.y * TM, col0 = blockIdx.x * bn;
    const int nk_all = (kdim + BK - 1) / BK;
    const int kb = epi.slabs_per_slice > 0 ? (int)blockIdx.z * epi.slabs_per_slice : 0;  // first k-slab of this slice
    const int nk = epi.slabs_per_slice > 0 ? min(nk_all - kb, epi.slabs_per_slice) : nk_all;
    const int chunk_len = CH > 0 ? CH : nk;

    if (threadIdx.x == 0) {
        for (int s = 0; s < RS; s++) mbar_init(raw_full + s, 1);
        for (int s = 0; s < L; s++) mbar_init(stage_done + s, 2);  // one commit from each MMA issuer
        for (int s = 0; s < DS; s++) mbar_init(conv_done + s, NCONV_WARPS);
        mbar_init(acc_full, 2);
        mbar_init(acc_empty, NCONV_WARPS);
        *abort_flag = 0;
        mbar_init_fence();
        prefetch_tmap(&tmA0);
        prefetch_tmap(&tmA1);
        prefetch_tmap(&tmB0);
        if (OP == OP_FWD) prefetch_tmap(&tmB1);
    }
    if (warp == 1) tmem_alloc(tmem_slot, NCOLS);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            for (int it = 0; it < nk; it++) {
                const int r = it % RS;
                if (it >= RS && !mbar_spin(stage_done + (it - RS) % L, ((it - RS) / L) & 1, abort_flag, status,
                                           ST_TIMEOUT_EMPTY))
                    break;
                mbar_arrive_expect_tx(raw_full + r, NRAW * TILE_BYTES);
                const uint32_t st = raw_base + r * NRAW * TILE_BYTES;
                const int k0 = (kb + it) * BK;
                load_tile<T::A_MN>(st + 0 * TILE_BYTES, &tmA0, row0, k0, raw_full + r);
                load_tile<T::A_MN>(st + 1 * TILE_BYTES, &tmA1, row0, k0, raw_full + r);
                load_tile<T::B_MN>(st + 2 * TILE_BYTES, &tmB0, col0, k0, raw_full + r);
                if (OP == OP_FWD) load_tile<T::B_MN>(st + 3 * TILE_BYTES, &tmB1, col0, k0, raw_full + r);
            }
        }
    } else if (warp == 1 || warp == ISSUER2_WARP) {
        // ------------------------------------------------------------------ MMA issuers: warp 1 -> D1, warp 10 -> D2
        if (lane == 0) {
            const bool chain1 = warp == 1;
            const uint32_t d1 = tmem, d2 = tmem + acc_stride;
            uint32_t f = 0;
            bool ok = true;
            for (int it = 0; it < nk && ok; it++) {
                const int r = it % RS, d = it % DS;
                if (it > 0 && it % chunk_len == 0) {
                    // the previous chunk must have been added to the register sums before it is overwritten
                    const int c = it / chunk_len;
                    ok = mbar_spin(acc_empty, (c - 1) & 1, abort_flag, status, ST_TIMEOUT_ACC);
                    if (!ok) break;
                    f = 0;
                }
                ok = mbar_spin(conv_done + d, (it / DS) & 1, abort_flag, status, ST_TIMEOUT_CONV);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t rs = raw_base + r * NRAW * TILE_BYTES, ds = der_base + d * NDER * TILE_BYTES;
                const uint32_t at = tmem + A_COL0 + d * (NA * BK);
                // descriptor words of raw B tile 0 (third tile of the raw slot) and derived B tile 0; k step j adds KSTEP
                constexpr uint32_t LBO = T::B_MN ? 2048 : 16, KSTEP = (T::B_MN ? 1024 : 32) >> 4;
                constexpr uint32_t HI = desc_hi(512, T::B_MN ? SWZ_128B_BASE32B : SWZ_64B);
                const uint32_t rbl = desc_lo(rs + 2 * TILE_BYTES, LBO), dsl = desc_lo(ds, LBO);
                if (chain1) {
                    mma_kstep_ts<OP == OP_FWD, 1>(d1, d2, at, rbl, dsl, HI, IDESC, f, f);
                    mma_kstep_ts<OP == OP_FWD, 1>(d1, d2, at + 8, rbl + KSTEP, dsl + KSTEP, HI, IDESC, 1, 1);
                } else {
                    mma_kstep_ts<OP == OP_FWD, 2>(d1, d2, at, rbl, dsl, HI, IDESC, f, f);
                    mma_kstep_ts<OP == OP_FWD, 2>(d1, d2, at + 8, rbl + KSTEP, dsl + KSTEP, HI, IDESC, 1, 1);
                }
                f = 1;
                mma_commit(stage_done + it % L);
                if (it % chunk_len == chunk_len - 1 || it == nk - 1) mma_commit(acc_full);
            }
        }
    } else if (warp >= 2 && warp < 2 + NCONV_WARPS) {  // warp 11 has no role in this kernel
        // ------------------------------------------------------------------ converters + accumulation + epilogue
        const int ct = threadIdx.x - 64;
        const int q = warp & 3;         // tensor-memory lane quadrant of this warp
        const int h = (warp - 2) >> 2;  // k step (A conversion) and column half (accumulation) of this warp
        const int arow = q * 32 + lane;  // A-tile row this thread converts
        const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16);
        float sum1[64], sum2[64];
#pragma unroll
        for (int i = 0; i < 64; i++) sum1[i] = sum2[i] = 0.f;

        auto drain = [&](int c) -> bool {
            if (!mbar_wait(acc_full, c & 1, abort_flag, status, ST_TIMEOUT_ACC)) return false;
            tc_fence_after_sync();
#pragma unroll
            for (int blk = 0; blk < 2; blk++) {
                float v[32];
                tmem_ld_32x32(lane_addr + h * 64 + blk * 32, v);
#pragma unroll
                for (int i = 0; i < 32; i++) sum1[blk * 32 + i] += v[i];
                tmem_ld_32x32(lane_addr + acc_stride + h * 64 + blk * 32, v);
#pragma unroll
                for (int i = 0; i < 32; i++) sum2[blk * 32 + i] += v[i];
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty);
            return true;
        };

        bool ok = true;
        int pending = -1;
        for (int it = 0; it < nk && ok; it++) {
            const int r = it % RS, d = it % DS;
            ok = mbar_wait(raw_full + r, (it / RS) & 1, abort_flag, status, ST_TIMEOUT_RAW) &&
                 (it < DS || mbar_wait(stage_done + (it - DS) % L, ((it - DS) / L) & 1, abort_flag, status,
                                       ST_TIMEOUT_EMPTY));
            if (!ok) break;
            const uint32_t rs = raw_base + r * NRAW * TILE_BYTES, ds = der_base + d * NDER * TILE_BYTES;

            // ---- A side: this thread's row, k step h (8 values) of both raw tiles -> tensor memory
            float a0[8], a1[8];
            if (T::A_MN) {
                // [32-row group][16 k rows][128 B], 32-byte atoms XOR-swizzled with the k row
                const uint32_t g = rs + q * 2048;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int k = h * 8 + i;
                    const uint32_t o = k * 128 + (((lane >> 3) ^ (k & 3)) << 5) + ((lane & 7) << 2);
                    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(a0[i]) : "r"(g + o));
                    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(a1[i]) : "r"(g + TILE_BYTES + o));
                }
            } else {
                // [128 rows][64 B], 16-byte chunks XOR-swizzled with (row / 2) % 4
                const uint32_t rowb = rs + arow * 64, sw = (arow >> 1) & 3;
                const float4 x0 = lds128(rowb + (((2 * h) ^ sw) << 4)), x1 = lds128(rowb + (((2 * h + 1) ^ sw) << 4));
                const float4 y0 = lds128(rowb + TILE_BYTES + (((2 * h) ^ sw) << 4));
                const float4 y1 = lds128(rowb + TILE_BYTES + (((2 * h + 1) ^ sw) << 4));
                a0[0] = x0.x, a0[1] = x0.y, a0[2] = x0.z, a0[3] = x0.w, a0[4] = x1.x, a0[5] = x1.y, a0[6] = x1.z, a0[7] = x1.w;
                a1[0] = y0.x, a1[1] = y0.y, a1[2] = y0.z, a1[3] = y0.w, a1[4] = y1.x, a1[5] = y1.y, a1[6] = y1.z, a1[7] = y1.w;
            }
            {
                const uint32_t at = lane_addr + A_COL0 + d * (NA * BK) + h * 8;
                float t0[8], t1[8];
#pragma unroll
                for (int i = 0; i < 8; i++) t0[i] = hi_part(a0[i]), t1[i] = hi_part(a1[i]);
                tmem_st_32x8(at + 0 * BK, t0);
                tmem_st_32x8(at + 1 * BK, t1);
#pragma unroll
                for (int i = 0; i < 8; i++) t0[i] = a0[i] - t0[i], t1[i] = a1[i] - t1[i];
                tmem_st_32x8(at + 2 * BK, t0);
                tmem_st_32x8(at + 3 * BK, t1);
                if (OP == OP_FWD) {
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const float sq = fmaf(a0[i], a0[i], a1[i]);
                        t0[i] = hi_part(sq);
                        t1[i] = sq - t0[i];
                    }
                    tmem_st_32x8(at + 4 * BK, t0);
                    tmem_st_32x8(at + 5 * BK, t1);
                }
            }
            // ---- B side: elementwise on 16-byte chunks, derived tiles at the same swizzled offsets
#pragma unroll
            for (int c = ct; c < CHUNKS; c += 32 * NCONV_WARPS) {
                const uint32_t o = c * 16;
                if (OP == OP_FWD) {
                    const float4 b0 = lds128(rs + 2 * TILE_BYTES + o), b1 = lds128(rs + 3 * TILE_BYTES + o);
                    const float4 qq = make_float4(b0.x * b0.x, b0.y * b0.y, b0.z * b0.z, b0.w * b0.w);
                    sts128(ds + 0 * TILE_BYTES + o, lo_part(b0));
                    sts128(ds + 1 * TILE_BYTES + o, lo_part(b1));
                    sts128(ds + 2 * TILE_BYTES + o, qq);
                    sts128(ds + 3 * TILE_BYTES + o, lo_part(qq));
                } else {
                    const float4 w = lds128(rs + 2 * TILE_BYTES + o);
                    const float4 qq = make_float4(w.x * w.x, w.y * w.y, w.z * w.z, w.w * w.w);
                    sts128(ds + 0 * TILE_BYTES + o, lo_part(w));
                    sts128(ds + 1 * TILE_BYTES + o, qq);
                    sts128(ds + 2 * TILE_BYTES + o, lo_part(qq));
                }
            }
            fence_proxy_async_smem();
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(conv_done + d);
            if (pending >= 0) {
                ok = drain(pending);
                pending = -1;
            }
            if (it % chunk_len == chunk_len - 1 || it == nk - 1) pending = it / chunk_len;
        }
        if (ok && pending >= 0) ok = drain(pending);

        if (ok) {
            const int row = row0 + q * 32 + lane;
            TcEpilogue e = epi;
            e.out1 += (long)blockIdx.z * epi.slice_elems;
            e.out2 += (long)blockIdx.z * epi.slice_elems;
            // all MMAs and TMA writes of this tile are complete (last acc_full phase): the operand rings are free
            if (e.npix > 0)
                store_tile<OP>(e, row, col0 + h * 64, bn - h * 64, sum1, sum2);
            else
                store_tile_staged<OP>(e, smem_base + (warp - 2) * STAGE_WARP, row - lane, lane, col0 + h * 64,
                                      bn - h * 64, sum1, sum2);
        }
    }
    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        if (*abort_flag) {
            const long long t0 = clock64();
            while (clock64() - t0 < 4000000LL) {
            }
        }
        tmem_dealloc(tmem, NCOLS);
    }
}

// =====================================================================================================
// Kernel "pair": as "ts", on CTA pairs (cta_group::2).
//
// The ts kernel still asks more of the shared-memory pipe per k-slab (tensor-core reads of B, converter traffic, TMA
// writes: about 1300 cycles' worth) than the MMAs take (about 1000 cycles), so it runs at the speed of shared memory.
// Here two CTAs of a cluster share one 256 x bn output tile: each keeps its own 128 rows of A (tensor memory) and of
// the accumulators, and only HALF of the B rows (bn / 2) in its shared memory; every MMA is one
// tcgen05.mma.cta_group::2 of 256 x bn x 8 issued by the even CTA, whose tensor cores on both SMs read each B half
// once. Per CTA that halves the B traffic of TMA, converters and tensor core. Barriers: TMA and ring-slot barriers are
// per CTA (the MMA's completion is multicast to both); "converted" and "accumulator drained" are counted in the
// issuing CTA, the other CTA's warps arrive there through the cluster's shared-memory window.
// =====================================================================================================

template <int OP, int RS, int DS>
constexpr size_t pair_smem_bytes() {
    return at_least_stage((size_t)RS * (2 * TILE_BYTES + PairTraits<OP>::NRAW_B * HALF_BYTES) +
                          (size_t)DS * PairTraits<OP>::NDER * HALF_BYTES) + 1024 + 256;
}

// FL bit 0 (GATHER): the A tiles of the forward / state pass are gathered inside the kernel (Conv2d, launched with 384
// threads); without it the kernel is launched with 352 threads and contains none of that code.
// FL bit 1 (RELU, forward only): the epilogue applies the ReLU and writes its Jacobian (TcEpilogue::out3).
// FL bit 2 (BIAS, parameter pass without a split contraction): the converter threads, which read every delta of their
// output feature anyway, also add them up; the pairs of the first column tile write the bias deltas.
template <int OP, int CH, int RS, int DS, int FL>
__global__ void __launch_bounds__(NTHREADS2, 1)
tagi_tc_linear_pair_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
                           const __grid_constant__ CUtensorMap tmB0, const __grid_constant__ CUtensorMap tmB1,
                           const TcEpilogue epi, const ConvGather cg, const int kdim, const int bn, int *status) {
    constexpr bool GATHER = (FL & 1) != 0, RELU = (FL & 2) != 0 && OP == OP_FWD;
    constexpr bool BIAS = (FL & 4) != 0 && OP == OP_BWD_PARAM;
    using T = OpTraits<OP>;
    using S = PairTraits<OP>;
    constexpr int NRAW_B = S::NRAW_B, NDER = S::NDER, NA = S::NA;
    constexpr uint32_t RAW_SLOT = 2 * TILE_BYTES + NRAW_B * HALF_BYTES, DER_SLOT = NDER * HALF_BYTES;
    constexpr uint32_t NCOLS = 512;
    // tensor-memory columns: D1 at 0, D2 at acc_stride, A tiles from 2 * acc_stride on (DS slots of NA * 16 columns)
    constexpr uint32_t acc_stride = (512 - DS * NA * BK) / 2 >= 128 ? 128 : 112;
    constexpr uint32_t A_COL0 = 2 * acc_stride;
    const uint32_t IDESC = make_idesc_tf32(256, bn, 0, T::B_MN);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *aligned = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t raw_base = smem_base, der_base = smem_base + RS * RAW_SLOT;
    // the epilogue stages its tile over the rings, so the barriers sit behind whichever is larger
    uint64_t *bars = reinterpret_cast<uint64_t *>(aligned + at_least_stage((size_t)RS * RAW_SLOT + (size_t)DS * DER_SLOT));
    constexpr int L = RS > DS ? RS : DS;  // stage_done ring, as in the one-CTA kernel; completion is multicast to both CTAs
    uint64_t *raw_full = bars, *stage_done = bars + RS, *conv_done = bars + RS + L;
    uint64_t *acc_full = bars + RS + L + DS, *acc_empty = acc_full + 1;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta = cluster_ctarank();  // 0 issues the MMAs
    const int half = bn / 2;
    const int row0 = blockIdx.y * 256 + (int)cta * 128;          // this CTA's 128 rows of A and of the output
    const int col0 = (blockIdx.x >> 1) * bn;                      // the pair's columns
    const int brow0 = col0 + (int)cta * half;                     // this CTA's half of the B rows
    const int nk_all = (kdim + BK - 1) / BK;
    const int kb = epi.slabs_per_slice > 0 ? (int)blockIdx.z * epi.slabs_per_slice : 0;  // first k-slab of this slice
    const int nk = epi.slabs_per_slice > 0 ? min(nk_all - kb, epi.slabs_per_slice) : nk_all;
    const int chunk_len = CH > 0 ? CH : nk;

    if (threadIdx.x == 0) {
        // one arrival from the TMA thread; with gathered A tiles one more from each of the 64 gathering threads
        for (int s = 0; s < RS; s++) mbar_init(raw_full + s, GATHER && cg.on ? 65 : 1);
        for (int s = 0; s < L; s++) mbar_init(stage_done + s, 2);  // one commit from each MMA issuer
        for (int s = 0; s < DS; s++) mbar_init(conv_done + s, NCONV_WARPS);  // used in CTA 0: one warp group of each CTA arrives
        mbar_init(acc_full, 2);
        mbar_init(acc_empty, 2 * NCONV_WARPS);          // used in CTA 0 only
        *abort_flag = 0;
        mbar_init_fence();
        if (!GATHER || !cg.on) {
            prefetch_tmap(&tmA0);
            prefetch_tmap(&tmA1);
        }
        prefetch_tmap(&tmB0);
        if (OP == OP_FWD) prefetch_tmap(&tmB1);
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot, NCOLS);
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers exist before anyone arrives on them
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (GATHER && cg.on && (warp == 0 || warp == GATHER_WARP)) {
        // ------------------------------------------------------------------ Conv2d: A tiles gathered with cp.async
        // Warps 0 and 11: each lane owns two of the CTA's 128 rows (pixels). The k index (channel, tap) is the same
        // for all lanes of an instruction, so consecutive lanes read consecutive pixels of one image row: coalesced.
        // Lane 0 of warp 0 also issues the TMA loads of the B tiles. Elements land in the 64-byte swizzle the
        // converter warps read (chunk c of row r at chunk c ^ ((r >> 1) & 3)).
        // The gather loop of these two warps paces the whole pipeline when tiles are narrow, so its per-element work is
        // kept minimal: the (channel, tap) of each of a slab's 16 k indices is worked out by one lane each and
        // broadcast, validity is one bit of a per-row tap mask, destination offsets are per-row constants.
        const int gw = warp == 0 ? 0 : 1;
        const int k2 = cg.k * cg.k;
        const long plane = (long)cg.H * cg.W;
        const float *base[2];
        unsigned long long tapmask[2];  // bit (ky * k + kx): that tap of the row's pixel lies inside the source image
        uint32_t relc[2][4];            // byte offset of 16-byte chunk c of the row inside an A tile (64-byte swizzle)
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int r = gw * 64 + j * 32 + lane;
            const long R = (long)row0 + r;
#pragma unroll
            for (int c = 0; c < 4; c++) relc[j][c] = r * 64 + ((c ^ ((r >> 1) & 3)) << 4);
            tapmask[j] = 0;
            base[j] = cg.s0;
            if (R < cg.rows) {
                const long bimg = R / cg.OHW;
                const int pp = (int)(R - bimg * cg.OHW), py = pp / cg.OW, px = pp - py * cg.OW;
                const int y0 = cg.sign > 0 ? py * cg.stride - cg.off : py + cg.off;
                const int x0 = cg.sign > 0 ? px * cg.stride - cg.off : px + cg.off;
                base[j] = cg.s0 + (bimg * cg.C * cg.H + y0) * cg.W + x0;
                for (int ty = 0; ty < cg.k; ty++)
                    for (int tx = 0; tx < cg.k; tx++)
                        if ((unsigned)(y0 + cg.sign * ty) < (unsigned)cg.H && (unsigned)(x0 + cg.sign * tx) < (unsigned)cg.W)
                            tapmask[j] |= 1ull << (ty * cg.k + tx);
            }
        }
        const long s1_off = cg.s1 - cg.s0;  // the second source has the same layout
        for (int it = 0; it < nk; it++) {
            const int r = it % RS;
            if (it >= RS && !mbar_wait(stage_done + (it - RS) % L, ((it - RS) / L) & 1, abort_flag, status, ST_TIMEOUT_EMPTY))
                break;
            const uint32_t st = raw_base + r * RAW_SLOT;
            if (warp == 0 && lane == 0) {
                mbar_arrive_expect_tx(raw_full + r, RAW_SLOT - 2 * TILE_BYTES);
                const int k0 = (kb + it) * BK;
                load_half_tile<T::B_MN>(st + 2 * TILE_BYTES, &tmB0, brow0, k0, raw_full + r);
                if (OP == OP_FWD) load_half_tile<T::B_MN>(st + 2 * TILE_BYTES + HALF_BYTES, &tmB1, brow0, k0, raw_full + r);
            }
            // lane j < 16 decodes k index j of this slab: element offset of (channel, tap) and the tap's mask bit
            int my_off = 0, my_tap = 63;  // bit 63 is never set: k indices past the contraction read zeros
            {
                const int kc = (kb + it) * BK + (lane & 15);
                if (kc < kdim) {
                    const int ci = kc / k2, t = kc - ci * k2, ky = t / cg.k, kx = t - ky * cg.k;
                    my_off = (int)(ci * plane) + cg.sign * (ky * cg.W + kx);
                    my_tap = t;
                }
            }
#pragma unroll
            for (int j16 = 0; j16 < BK; j16++) {
                const int off = __shfl_sync(0xffffffffu, my_off, j16), tap = __shfl_sync(0xffffffffu, my_tap, j16);
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const bool v = (tapmask[j] >> tap) & 1ull;
                    const float *src = v ? base[j] + off : cg.s0;
                    const uint32_t d = st + relc[j][j16 >> 2] + ((j16 & 3) << 2);
                    cp_async_f32(d, src, v);
                    cp_async_f32(d + TILE_BYTES, src + s1_off, v);
                }
            }
            cp_async_arrive(raw_full + r);
        }
        cp_async_wait_all();
    } else if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (each CTA for itself)
        if (lane == 0) {
            for (int it = 0; it < nk; it++) {
                const int r = it % RS;
                if (it >= RS && !mbar_wait(stage_done + (it - RS) % L, ((it - RS) / L) & 1, abort_flag, status,
                                           ST_TIMEOUT_EMPTY))
                    break;
                mbar_arrive_expect_tx(raw_full + r, RAW_SLOT);
                const uint32_t st = raw_base + r * RAW_SLOT;
                const int k0 = (kb + it) * BK;
                load_tile<T::A_MN>(st, &tmA0, row0, k0, raw_full + r);
                load_tile<T::A_MN>(st + TILE_BYTES, &tmA1, row0, k0, raw_full + r);
                load_half_tile<T::B_MN>(st + 2 * TILE_BYTES, &tmB0, brow0, k0, raw_full + r);
                if (OP == OP_FWD) load_half_tile<T::B_MN>(st + 2 * TILE_BYTES + HALF_BYTES, &tmB1, brow0, k0, raw_full + r);
            }
        }
    } else if (warp == 1 || warp == ISSUER2_WARP) {
        // ------------------------------------------------------------------ MMA issuers (CTA 0): warp 1 -> D1, warp 10 -> D2
        if (lane == 0 && cta == 0) {
            const bool chain1 = warp == 1;
            const uint32_t d1 = tmem, d2 = tmem + acc_stride;
            uint32_t f = 0;
            bool ok = true;
            for (int it = 0; it < nk && ok; it++) {
                const int r = it % RS, d = it % DS;
                if (it > 0 && it % chunk_len == 0) {
                    const int c = it / chunk_len;
                    ok = mbar_wait_cluster(acc_empty, (c - 1) & 1, abort_flag, status, ST_TIMEOUT_ACC);
                    if (!ok) break;
                    f = 0;
                }
                ok = mbar_wait_cluster(conv_done + d, (it / DS) & 1, abort_flag, status, ST_TIMEOUT_CONV);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t rb = raw_base + r * RAW_SLOT + 2 * TILE_BYTES, ds = der_base + d * DER_SLOT;
                const uint32_t at = tmem + A_COL0 + d * (NA * BK);
                constexpr uint32_t LBO = T::B_MN ? 2048 : 16, KSTEP = (T::B_MN ? 1024 : 32) >> 4;
                constexpr uint32_t HI = desc_hi(512, T::B_MN ? SWZ_128B_BASE32B : SWZ_64B);
                const uint32_t rbl = desc_lo(rb, LBO), dsl = desc_lo(ds, LBO);
                if (chain1) {
                    mma_kstep_pair<OP == OP_FWD, 1>(d1, d2, at, rbl, dsl, HI, IDESC, f, f);
                    mma_kstep_pair<OP == OP_FWD, 1>(d1, d2, at + 8, rbl + KSTEP, dsl + KSTEP, HI, IDESC, 1, 1);
                } else {
                    mma_kstep_pair<OP == OP_FWD, 2>(d1, d2, at, rbl, dsl, HI, IDESC, f, f);
                    mma_kstep_pair<OP == OP_FWD, 2>(d1, d2, at + 8, rbl + KSTEP, dsl + KSTEP, HI, IDESC, 1, 1);
                }
                f = 1;
                mma_commit_pair(stage_done + it % L);  // both CTAs may refill the raw slot and overwrite the derived one
                if (it % chunk_len == chunk_len - 1 || it == nk - 1) mma_commit_pair(acc_full);
            }
        }
    } else if (warp >= 2 && warp < 2 + NCONV_WARPS) {
        // ------------------------------------------------------------------ converters + accumulation + epilogue
        const int ct = threadIdx.x - 64;
        const int q = warp & 3;
        const int h = (warp - 2) >> 2;
        const int arow = q * 32 + lane;
        const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16);
        float sum1[64], sum2[64];
#pragma unroll
        for (int i = 0; i < 64; i++) sum1[i] = sum2[i] = 0.f;
        float bsum0 = 0.f, bsum1 = 0.f;  // BIAS: sums of this thread's row of the two A operands over its k-slabs

        auto drain = [&](int c) -> bool {
            if (!mbar_wait(acc_full, c & 1, abort_flag, status, ST_TIMEOUT_ACC)) return false;
            tc_fence_after_sync();
#pragma unroll
            for (int blk = 0; blk < 2; blk++) {
                float v[32];
                tmem_ld_32x32(lane_addr + h * 64 + blk * 32, v);
#pragma unroll
                for (int i = 0; i < 32; i++) sum1[blk * 32 + i] += v[i];
                tmem_ld_32x32(lane_addr + acc_stride + h * 64 + blk * 32, v);
#pragma unroll
                for (int i = 0; i < 32; i++) sum2[blk * 32 + i] += v[i];
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty, 0);
            return true;
        };

        // The converter warps work as two groups of four (h = 0 / 1) on alternate k-slabs, so that two slabs are being
        // converted at any time: one slab's conversion is a chain of shared-memory loads, tcgen05.st, fences and a
        // barrier arrive whose latency, not its instruction count, set the pace when all eight warps shared one slab.
        bool ok = true;
        int pending = -1;  // chunk whose MMAs may be issued and whose sums this warp has not collected yet
        int scanned = 0;   // slabs below this index have been checked for chunk ends
        auto note_chunk_ends = [&](int upto) {  // slabs scanned .. upto
            for (int sl = scanned; sl <= upto && sl < nk && ok; sl++)
                if (sl % chunk_len == chunk_len - 1 || sl == nk - 1) {
                    if (pending >= 0) ok = drain(pending);
                    pending = sl / chunk_len;
                }
            scanned = upto + 1;
        };
        const int gt = ct & 127;  // thread index inside the group
        for (int it = h; it < nk && ok; it += 2) {
            const int r = it % RS, d = it % DS;
            ok = mbar_wait(raw_full + r, (it / RS) & 1, abort_flag, status, ST_TIMEOUT_RAW) &&
                 (it < DS || mbar_wait(stage_done + (it - DS) % L, ((it - DS) / L) & 1, abort_flag, status,
                                       ST_TIMEOUT_EMPTY));
            if (!ok) break;
            const uint32_t rs = raw_base + r * RAW_SLOT, rb = rs + 2 * TILE_BYTES, ds = der_base + d * DER_SLOT;

#pragma unroll
            for (int kh = 0; kh < 2; kh++) {  // the two 8-wide k steps of the A tiles: this thread's row
                float a0[8], a1[8];
                if (T::A_MN) {
                    const uint32_t g = rs + q * 2048;
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const int kk = kh * 8 + i;
                        const uint32_t o = kk * 128 + (((lane >> 3) ^ (kk & 3)) << 5) + ((lane & 7) << 2);
                        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(a0[i]) : "r"(g + o));
                        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(a1[i]) : "r"(g + TILE_BYTES + o));
                    }
                } else {
                    const uint32_t rowb = rs + arow * 64, sw = (arow >> 1) & 3;
                    const float4 x0 = lds128(rowb + (((2 * kh) ^ sw) << 4)), x1 = lds128(rowb + (((2 * kh + 1) ^ sw) << 4));
                    const float4 y0 = lds128(rowb + TILE_BYTES + (((2 * kh) ^ sw) << 4));
                    const float4 y1 = lds128(rowb + TILE_BYTES + (((2 * kh + 1) ^ sw) << 4));
                    a0[0] = x0.x, a0[1] = x0.y, a0[2] = x0.z, a0[3] = x0.w, a0[4] = x1.x, a0[5] = x1.y, a0[6] = x1.z, a0[7] = x1.w;
                    a1[0] = y0.x, a1[1] = y0.y, a1[2] = y0.z, a1[3] = y0.w, a1[4] = y1.x, a1[5] = y1.y, a1[6] = y1.z, a1[7] = y1.w;
                }
                if (BIAS) {
#pragma unroll
                    for (int i = 0; i < 8; i++) bsum0 += a0[i], bsum1 += a1[i];
                }
                const uint32_t at = lane_addr + A_COL0 + d * (NA * BK) + kh * 8;
                float t0[8], t1[8];
#pragma unroll
                for (int i = 0; i < 8; i++) t0[i] = hi_part(a0[i]), t1[i] = hi_part(a1[i]);
                tmem_st_32x8(at + 0 * BK, t0);
                tmem_st_32x8(at + 1 * BK, t1);
#pragma unroll
                for (int i = 0; i < 8; i++) t0[i] = a0[i] - t0[i], t1[i] = a1[i] - t1[i];
                tmem_st_32x8(at + 2 * BK, t0);
                tmem_st_32x8(at + 3 * BK, t1);
                if (OP == OP_FWD) {
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const float sq = fmaf(a0[i], a0[i], a1[i]);
                        t0[i] = hi_part(sq);
                        t1[i] = sq - t0[i];
                    }
                    tmem_st_32x8(at + 4 * BK, t0);
                    tmem_st_32x8(at + 5 * BK, t1);
                }
            }
            // B halves: two 16-byte chunks per thread of the group
#pragma unroll
            for (int c = 0; c < 2; c++) {
                const uint32_t o = gt * 16 + c * (HALF_BYTES / 2);
                if (OP == OP_FWD) {
                    const float4 b0 = lds128(rb + o), b1 = lds128(rb + HALF_BYTES + o);
                    const float4 qq = make_float4(b0.x * b0.x, b0.y * b0.y, b0.z * b0.z, b0.w * b0.w);
                    sts128(ds + 0 * HALF_BYTES + o, lo_part(b0));
                    sts128(ds + 1 * HALF_BYTES + o, lo_part(b1));
                    sts128(ds + 2 * HALF_BYTES + o, qq);
                    sts128(ds + 3 * HALF_BYTES + o, lo_part(qq));
                } else {
                    const float4 w = lds128(rb + o);
                    const float4 qq = make_float4(w.x * w.x, w.y * w.y, w.z * w.z, w.w * w.w);
                    sts128(ds + 0 * HALF_BYTES + o, lo_part(w));
                    sts128(ds + 1 * HALF_BYTES + o, qq);
                    sts128(ds + 2 * HALF_BYTES + o, lo_part(qq));
                }
            }
            fence_proxy_async_smem();
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(conv_done + d, 0);
            if (pending >= 0) {
                ok = drain(pending);
                pending = -1;
            }
            note_chunk_ends(it + 1);
        }
        if (ok) note_chunk_ends(nk - 1);
        if (ok && pending >= 0) ok = drain(pending);

        if (BIAS) {
            // the two converter groups took alternate k-slabs: group 1 hands its sums over through shared memory behind
            // the epilogue's staging area (inside the operand rings, which are idle by now)
            static_assert(!BIAS || (size_t)RS * RAW_SLOT + (size_t)DS * DER_SLOT >= STAGE_BYTES + 128 * 8,
                          "no room for the bias hand-over behind the staging area");
            const uint32_t slot = smem_base + (uint32_t)STAGE_BYTES + arow * 8;
            if (h == 1 && ok) asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(slot), "f"(bsum0), "f"(bsum1) : "memory");
            asm volatile("bar.sync 1, %0;" ::"n"(NCONV_WARPS * 32) : "memory");
            const int row = row0 + arow;
            if (h == 0 && ok && col0 == 0 && row < epi.rows) {
                float p0, p1;
                asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(p0), "=f"(p1) : "r"(slot));
                const float vb = __ldg(epi.aux2 + row);
                epi.bias1[row] = (bsum0 + p0) * vb;
                epi.bias2[row] = (bsum1 + p1) * vb * vb;
            }
        }
        if (ok) {
            const int row = row0 + q * 32 + lane;
            TcEpilogue e = epi;
            e.out1 += (long)blockIdx.z * epi.slice_elems;
            e.out2 += (long)blockIdx.z * epi.slice_elems;
            // all MMAs and TMA writes of this tile are complete (last acc_full phase): the operand rings are free
            if (e.npix > 0)
                store_tile<OP, RELU>(e, row, col0 + h * 64, bn - h * 64, sum1, sum2);
            else
                store_tile_staged<OP, RELU>(e, smem_base + (warp - 2) * STAGE_WARP, row - lane, lane, col0 + h * 64,
                                            bn - h * 64, sum1, sum2);
        }
    }
    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // neither CTA leaves (or frees tensor memory) while the other may still signal or read it
    if (warp == 1) {
        if (*abort_flag) {
            const long long t0 = clock64();
            while (clock64() - t0 < 4000000LL) {
            }
        }
        tmem_dealloc_pair(tmem, NCOLS);
    }
}

// ------------------------------------------------------------------------------------------- host side
EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Tensor map over a row-major FP32 matrix [outer][inner]. K-major operand tiles: box 16 x 128, 64-byte
// swizzle; MN-major: box 32 x 16, 128-byte swizzle with 32-byte atoms.
int make_tmap(CUtensorMap *tm, const float *ptr, uint64_t inner, uint64_t outer, bool mn_major, unsigned kmajor_rows = 128,
              uint64_t pitch = 0) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(TAGI_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {(pitch ? pitch : inner) * sizeof(float)};
    cuuint32_t box[2] = {mn_major ? 32u : (cuuint32_t)BK, mn_major ? (cuuint32_t)BK : (cuuint32_t)kmajor_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE,
                    mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_64B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(TAGI_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
    return TAGI_OK;
}

int *status_word() {
    static int *ptr[64] = {};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(mu);
    if (!ptr[dev]) {
        if (cudaMalloc(&ptr[dev], sizeof(int)) != cudaSuccess) return nullptr;
        cudaMemset(ptr[dev], 0, sizeof(int));
    }
    return ptr[dev];
}

std::atomic<int> g_variant{3};  // 3: CTA pairs (default; passes with < 256 output rows use 1); 1: one CTA per tile everywhere
int g_pair_bn = 0;  // forces the pair kernel's tile width (diagnostic); 0 = chosen per launch
std::atomic<int> g_sms{148};    // SMs the tile planning counts on (tagi_tc_set_sm_budget)
std::atomic<int> g_chunked{1};  // 1: contraction accumulated in chunks of 256 (default); 0: one accumulation chain (diagnostic)

template <int OP>
int launch(const CUtensorMap &a0, const CUtensorMap &a1, const CUtensorMap &b0, const CUtensorMap &b1,
           const TcEpilogue &epi, int kdim, cudaStream_t st) {
    int *status = status_word();
    if (!status) return fail(TAGI_ERR_CUDA, "cannot allocate the tensor-core status word");
    // Columns per tile: the width (a multiple of 16 up to 128) that minimises waves-of-148-CTAs x width, i.e. the
    // tensor-core time of the slowest SM; e.g. 4096 columns x 8 row tiles run as 296 tiles of 112 (two full waves)
    // rather than 256 tiles of 128 (two waves, the second 73 % full).
    const long row_tiles = (epi.rows + TM - 1) / TM;
    const long sms = g_sms;   // read once: another host thread may change the budget while this call plans
    int bn = TN;
    long best = -1;
    for (int w = TN; w >= 64; w -= 16) {
        const long tiles = row_tiles * ((epi.cols + w - 1) / w);
        const long cost = ((tiles + sms - 1) / sms) * (w + 16);  // + 16: per-tile work that does not shrink with the width
        if (best < 0 || cost < best) best = cost, bn = w;
    }
    const unsigned slices = epi.slabs_per_slice > 0 ? (unsigned)(((kdim + BK - 1) / BK + epi.slabs_per_slice - 1) / epi.slabs_per_slice) : 1u;
    dim3 grid((epi.cols + bn - 1) / bn, (unsigned)row_tiles, slices);
    cudaError_t e;
    // ring depths: four raw slots, two derived slots (what the forward pass's six A tiles per slot leave of tensor memory)
#define TAGI_TS_LAUNCH(CHV)                                                                                      \
    do {                                                                                                         \
        auto k = tagi_tc_linear_ts_kernel<OP, CHV, 4, 2>;                                                        \
        constexpr size_t sm = ts_smem_bytes<OP, 4, 2>();                                                         \
        e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);                       \
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute");                                       \
        k<<<grid, NTHREADS2, sm, st>>>(a0, a1, b0, b1, epi, kdim, bn, status);                                   \
    } while (0)
    if (g_chunked) TAGI_TS_LAUNCH(CHUNK_STAGES); else TAGI_TS_LAUNCH(0);
#undef TAGI_TS_LAUNCH
    e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "tensor-core Linear kernel launch");
    return TAGI_OK;
}

// CTA-pair variant: grid.x = 2 x column tiles (cluster of two along x), grid.y = 256-row tiles.
template <int OP>
int launch_pair(const CUtensorMap &a0, const CUtensorMap &a1, const CUtensorMap &b0, const CUtensorMap &b1,
                const TcEpilogue &epi, int kdim, cudaStream_t st, const ConvGather &cg = ConvGather{}) {
    int *status = status_word();
    if (!status) return fail(TAGI_ERR_CUDA, "cannot allocate the tensor-core status word");
    const long row_tiles = (epi.rows + 255) / 256;
    const long sms = g_sms;   // read once: another host thread may change the budget while this call plans
    int bn = TN;
    long best = -1;
    for (int w = TN; w >= 64; w -= 16) {  // 74 pairs run at a time
        const long tiles = row_tiles * ((epi.cols + w - 1) / w);
        const long cost = ((tiles + sms / 2 - 1) / (sms / 2)) * (w + 16);
        if (best < 0 || cost < best) best = cost, bn = w;
    }
    if (g_pair_bn) bn = g_pair_bn;
    cudaLaunchConfig_t cfg = {};
    const unsigned slices = epi.slabs_per_slice > 0 ? (unsigned)(((kdim + BK - 1) / BK + epi.slabs_per_slice - 1) / epi.slabs_per_slice) : 1u;
    cfg.gridDim = dim3(2 * (unsigned)((epi.cols + bn - 1) / bn), (unsigned)row_tiles, slices);
    cfg.blockDim = dim3(NTHREADS2);
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    cudaError_t e;
#define TAGI_PAIR_LAUNCH_G(CHV, RSV, DSV, GV)                                                  \
    do {                                                                                         \
        auto k = tagi_tc_linear_pair_kernel<OP, CHV, RSV, DSV, GV>;                              \
        constexpr size_t sm = pair_smem_bytes<OP, RSV, DSV>();                                   \
        cfg.dynamicSmemBytes = sm;                                                               \
        cfg.blockDim = dim3(((GV) & 1) ? NTHREADS2 : NTHREADS2 - 32);                            \
        e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);       \
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute");                       \
        e = cudaLaunchKernelEx(&cfg, k, a0, a1, b0, b1, epi, cg, kdim, bn, status);              \
    } while (0)
#define TAGI_PAIR_LAUNCH(CHV, RSV, DSV)                                                                  \
    do {                                                                                                   \
        constexpr int G = OP != OP_BWD_PARAM ? 1 : 0, R = OP == OP_FWD ? 2 : 0;                            \
        const bool gather = OP != OP_BWD_PARAM && cg.on, relu = OP == OP_FWD && epi.out3 != nullptr;       \
        if (OP == OP_BWD_PARAM && epi.bias1 != nullptr) TAGI_PAIR_LAUNCH_G(CHV, RSV, DSV, 4 - G * 4);      \
        else if (gather && relu) TAGI_PAIR_LAUNCH_G(CHV, RSV, DSV, G | R);                                 \
        else if (gather) TAGI_PAIR_LAUNCH_G(CHV, RSV, DSV, G);                                             \
        else if (relu) TAGI_PAIR_LAUNCH_G(CHV, RSV, DSV, R);                                               \
        else TAGI_PAIR_LAUNCH_G(CHV, RSV, DSV, 0);                                                         \
    } while (0)
    // ring depths: hand-offs cross two SMs here, so the derived ring is as deep as tensor memory allows (backward:
    // four slots; forward: three when the accumulators fit 2 x 112 columns, else two)
    if constexpr (OP == OP_FWD) {
        if (bn <= 112) {
            if (g_chunked) TAGI_PAIR_LAUNCH(CHUNK_STAGES, 5, 3); else TAGI_PAIR_LAUNCH(0, 5, 3);
        } else {
            if (g_chunked) TAGI_PAIR_LAUNCH(CHUNK_STAGES, 5, 2); else TAGI_PAIR_LAUNCH(0, 5, 2);
        }
    } else {
        if (g_chunked) TAGI_PAIR_LAUNCH(CHUNK_STAGES, 6, 4); else TAGI_PAIR_LAUNCH(0, 6, 4);
    }
#undef TAGI_PAIR_LAUNCH
#undef TAGI_PAIR_LAUNCH_G
    if (e != cudaSuccess) return cuda_fail(e, "tensor-core Linear pair kernel launch");
    return TAGI_OK;
}

// the pair kernel needs at least one full 256-row tile to pay off
inline bool use_pair(int rows) { return g_variant == 3 && rows >= 256; }

}  // namespace

EncodeTiledFn tc_encode_fn() { return encode_fn(); }
int *tc_status_word() { return status_word(); }
int tc_sm_budget() { return g_sms; }
int tc_chunked() { return g_chunked; }

// Shapes the tensor-core path takes: 16-byte aligned tensors, every dimension a multiple of 4 (TMA pitches
// and vector stores), and large enough for 128 x 128 tiles to make sense.
bool linear_tc_supported(int B, int K, int N, std::initializer_list<const void *> ptrs) {
    if (B % 4 || K % 4 || N % 4) return false;
    for (const void *p : ptrs)
        if (p && !aligned16(p)) return false;
    return true;
}
bool linear_tc_profitable(int B, int K, int N) { return B >= 128 && K >= 128 && N >= 128; }

int linear_tc_set_variant(int v) {
    if (!(v == 1 || v == 3 || (v >= 64 && v <= 128 && v % 16 == 0)))
        return fail(TAGI_ERR_INVALID_ARGUMENT, "variant must be 3 (CTA pairs), 1 (one CTA per tile) or a pair tile width "
                                               "64, 80, 96, 112, 128");
    if (v >= 64) {  // CTA pairs with this tile width (diagnostic)
        g_pair_bn = v;
        v = 3;
    } else {
        g_pair_bn = 0;
    }
    g_variant = v;
    return TAGI_OK;
}
int linear_tc_set_sm_budget(int sms) {
    if (sms != 0 && (sms < 2 || sms > 148)) return fail(TAGI_ERR_INVALID_ARGUMENT, "SM budget must be 0 (all) or 2 .. 148");
    g_sms = sms == 0 ? 148 : sms;
    return TAGI_OK;
}
int linear_tc_set_chunked(int on) {
    g_chunked = on ? 1 : 0;
    return TAGI_OK;
}

int linear_tc_status(int *out, int reset) {
    int *w = status_word();
    if (!w) return fail(TAGI_ERR_CUDA, "no status word");
    cudaError_t e = cudaMemcpy(out, w, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpy(status)");
    if (reset && *out) cudaMemset(w, 0, sizeof(int));
    return TAGI_OK;
}

int linear_fwd_tc(const float *mu_w, const float *var_w, const float *mu_b, const float *var_b, const float *mu_a,
                  const float *var_a, int B, int K, int N, float *mu_z, float *var_z, cudaStream_t st, int npix,
                  const ConvGather *cg, float *relu_jcb) {
    CUtensorMap a0, a1, b0, b1;
    int rc;
    const bool pair = use_pair(B);
    if ((rc = make_tmap(&b0, mu_w, K, N, false, pair ? 64 : 128))) return rc;
    if ((rc = make_tmap(&b1, var_w, K, N, false, pair ? 64 : 128))) return rc;
    // relu_jcb: the ReLU is applied in the epilogue (CTA-pair kernel only): mu_z / var_z receive the moments after it
    if (relu_jcb && !pair) return fail(TAGI_ERR_UNSUPPORTED, "the fused ReLU needs the CTA-pair kernel");
    TcEpilogue epi{mu_z, var_z, mu_b, var_b, (long)N, B, N, npix, 0, 0, relu_jcb};
    if (cg) {  // A = the receptive fields of (mu_a, var_a), gathered inside the kernel
        if (!pair) return fail(TAGI_ERR_UNSUPPORTED, "implicit Conv2d operands need the CTA-pair kernel");
        return launch_pair<OP_FWD>(b0, b0, b0, b1, epi, K, st, *cg);
    }
    if ((rc = make_tmap(&a0, mu_a, K, B, false))) return rc;
    if ((rc = make_tmap(&a1, var_a, K, B, false))) return rc;
    if (pair) return launch_pair<OP_FWD>(a0, a1, b0, b1, epi, K, st);
    return launch<OP_FWD>(a0, a1, b0, b1, epi, K, st);
}
bool linear_tc_pair_for(int rows) { return use_pair(rows); }
bool linear_bwd_param_tc_fuses_bias(int N) { return use_pair(N); }

int linear_bwd_state_tc(const float *mu_w, const float *jcb, const float *dmu_z, const float *dvar_z, int B, int K,
                        int N, float *dmu_a, float *dvar_a, cudaStream_t st, int npix, const ConvGather *cg) {
    // rows = batch, columns = input features, contraction over output features; mu_w [N][K] is MN-major here
    CUtensorMap a0, a1, b0;
    int rc;
    if ((rc = make_tmap(&b0, mu_w, K, N, true))) return rc;
    TcEpilogue epi{dmu_a, dvar_a, jcb, nullptr, (long)K, B, K, npix, 0, 0};
    if (cg) {  // A = the deltas each input pixel receives, gathered inside the kernel
        if (!use_pair(B)) return fail(TAGI_ERR_UNSUPPORTED, "implicit Conv2d operands need the CTA-pair kernel");
        return launch_pair<OP_BWD_STATE>(b0, b0, b0, b0, epi, N, st, *cg);
    }
    if ((rc = make_tmap(&a0, dmu_z, N, B, false))) return rc;
    if ((rc = make_tmap(&a1, dvar_z, N, B, false))) return rc;
    if (use_pair(B)) return launch_pair<OP_BWD_STATE>(a0, a1, b0, b0, epi, N, st);
    return launch<OP_BWD_STATE>(a0, a1, b0, b0, epi, N, st);
}

// Sum of the contraction slices in slice order, then the scaling of the parameter pass (s and s*s)
__global__ void __launch_bounds__(256) tc_reduce_slices_kernel(const float *__restrict__ part1, const float *__restrict__ part2,
                                                               const float *__restrict__ scale, long n, int slices,
                                                               float *__restrict__ out1, float *__restrict__ out2) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float a1 = 0.f, a2 = 0.f;
    for (int z = 0; z < slices; z++) {
        a1 += part1[(long)z * n + i];
        a2 += part2[(long)z * n + i];
    }
    const float sc = __ldg(scale + i);
    out1[i] = a1 * sc;
    out2[i] = a2 * sc * sc;
}

// How many slices the contraction (B long) of a parameter pass with an N x K output should be cut into: none when the
// output tiles already fill half the SMs, else about two waves of CTAs, keeping at least 64 k-slabs (1024 batch rows)
// per slice. 1 = do not split.
int linear_bwd_param_tc_slices(int B, int K, int N) {
    const long tiles = (long)((N + 127) / 128) * ((K + 127) / 128);
    const int nk = (B + BK - 1) / BK;
    if (tiles > 74) return 1;
    long s = (2 * 148 + tiles - 1) / tiles;
    if (s > nk / 64) s = nk / 64;
    return s < 2 ? 1 : (int)s;
}

// split_ws: optional scratch of at least 2 * slices * N * K floats (slices from linear_bwd_param_tc_slices); without it
// the contraction is not split.
int linear_bwd_param_tc(const float *var_w, const float *mu_a, const float *dmu_z, const float *dvar_z, int B, int K,
                        int N, float *dmu_w, float *dvar_w, cudaStream_t st, float *split_ws, int slices, long ldz,
                        const float *var_b, float *dmu_b, float *dvar_b) {
    // rows = output features, columns = input features, contraction over the batch; both operands MN-major.
    // ldz: row pitch of the delta matrices (0 = N; larger when only a range of the output features is computed)
    CUtensorMap a0, a1, b0;
    int rc;
    if ((rc = make_tmap(&a0, dmu_z, N, B, true, 128, ldz))) return rc;
    if ((rc = make_tmap(&a1, dvar_z, N, B, true, 128, ldz))) return rc;
    if ((rc = make_tmap(&b0, mu_a, K, B, true))) return rc;
    if (!split_ws || slices < 2) {
        TcEpilogue epi{dmu_w, dvar_w, var_w, nullptr, (long)K, N, K, 0, 0, 0};
        if (use_pair(N)) {
            // var_b: the bias deltas come out of the same kernel (see linear_bwd_param_tc_fuses_bias)
            if (var_b) epi.aux2 = var_b, epi.bias1 = dmu_b, epi.bias2 = dvar_b;
            return launch_pair<OP_BWD_PARAM>(a0, a1, b0, b0, epi, B, st);
        }
        if (var_b) return fail(TAGI_ERR_UNSUPPORTED, "bias deltas are folded into the CTA-pair kernel only");
        return launch<OP_BWD_PARAM>(a0, a1, b0, b0, epi, B, st);
    }
    const long slice = (long)N * K;
    const int nk = (B + BK - 1) / BK;
    const int per = (nk + slices - 1) / slices;
    const int used = (nk + per - 1) / per;
    float *p1 = split_ws, *p2 = split_ws + (long)slices * slice;
    TcEpilogue epi{p1, p2, nullptr, nullptr, (long)K, N, K, 0, per, slice};
    rc = use_pair(N) ? launch_pair<OP_BWD_PARAM>(a0, a1, b0, b0, epi, B, st)
                     : launch<OP_BWD_PARAM>(a0, a1, b0, b0, epi, B, st);
    if (rc != TAGI_OK) return rc;
    tc_reduce_slices_kernel<<<(unsigned)((slice + 255) / 256), 256, 0, st>>>(p1, p2, var_w, slice, used, dmu_w, dvar_w);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "tc_reduce_slices_kernel launch");
    return TAGI_OK;
}

}  // namespace tagi
