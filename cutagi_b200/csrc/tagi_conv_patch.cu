// TAGI Conv2d parameter pass as an implicit GEMM on the tensor cores (tcgen05 cta_group::2, 3xTF32): no im2col matrix
// and no regrouped deltas ever exist in memory.
//
//   dmu_w [co][ci, ky, kx] = var_w   * sum over (b, oy, ox) of dmu_z [b][co][oy][ox] * mu_a[b][ci][oy*s - off + ky][ox*s - off + kx]
//   dvar_w[co][ci, ky, kx] = var_w^2 * sum ...              of dvar_z[b][co][oy][ox] * mu_a[...]^2
// (CPU definition: conv2d_bwd_delta_w, src/conv2d_layer.cpp:459-494 of cuTAGI).
//
// GEMM view, with the roles chosen so that both operands are read as they lie in memory:
//   rows (A side, tensor memory)  = weight columns (ci, ky, kx) in their natural order; a CTA owns CT channels x k*k taps
//                                   (CT * k * k <= 128 rows), a CTA pair two such tiles
//   columns (B side, shared mem.) = output channels co; the deltas [b][co][oy][ox] are K-major for this GEMM as they are
//   contraction                   = output pixels, 16 at a time: one slab is (image b, output row oy, columns ox0..ox0+15)
// Per slab the producer thread issues three TMA box copies:
//   * the input patch of the CTA's channels: box [PW columns][k rows][CT channels][1 image] of mu_a starting at
//     (ox0*s - off rounded down to a 16-byte boundary, oy*s - off, c0, b); out-of-image coordinates arrive as zeros, which
//     is exactly the padding rule (src/indices.cpp:63-104), so no masks exist anywhere;
//   * the two delta tiles: box [16 pixels][1 row][64 channels][1 image] of dmu_z and dvar_z in the 64-byte swizzle the
//     tensor core reads. Pixels past the end of the output row arrive as zeros, so whatever the patch holds there is
//     multiplied by zero.
// The converter thread of row (c, ky, kx) reads its 16 values from the patch at (c, ky, kx + lead + i*s), i = 0..15, forms
// x, x^2 and their TF32 hi / lo parts and writes them to tensor memory; another part of the same threads derives the lo
// tiles of the deltas. The MMAs, the chunked accumulation (256 contraction steps per chunk, summed in FP32 registers)
// and the barriers between the roles are those of the Linear CTA-pair kernel (tagi_linear_tc.cu).
// The output is small (fo x fi*k*k) and the contraction long (B * ho * ceil(wo/16) slabs), so the slabs are cut into
// slices across CTA pairs; slices go to scratch and are summed in slice order (results do not depend on scheduling).
//
// Flat mode, for images whose rows are not a multiple of 16 bytes (14 x 14) but whose planes are: TMA cannot address image
// rows then, so an image plane is treated as one row of H*W pixels (stride-1 layers that keep the image size). A slab is
// 16 consecutive pixels p0..p0+15 of the flattened plane, its patch the run [p0 - halo, p0 + 16 + halo) of each channel,
// and tap (ky, kx) of pixel p is the patch entry p + (ky - off) * W + (kx - off). Entries whose column leaves the image row
// belong to the neighbouring row instead of the padding; the converter thread sets them to zero (the column of pixel i is
// (p0 + i) mod W). Rows above and below the image fall outside the plane and arrive as zeros as before.
#include "tagi_tc_tile.cuh"

namespace tagi {
namespace {

struct PatchParam {
    int fi, k, k2, Kc, fo;
    int CT;               // channels per CTA row tile
    int ho, nxc;          // output rows per image, slabs (chunks of 16 or 32 pixels) per output row
    int stride, PW, lead; // patch row pitch in floats; a row's first useful column
    int x0, y0;           // patch origin relative to (ox0 * stride, oy * stride): -(off + lead), -off
    int total_slabs, slabs_per_slice;
    uint32_t a_bytes;     // bytes of the patch box
    uint32_t a_slot;      // ring slot reserved for it (multiple of 1024)
    float *out1, *out2;   // [slice][fo][Kc]
    const float *scale;   // var_w when the contraction is not sliced, else null (raw partial sums)
    long slice_elems;
    int flat, W, off;     // flat mode (see above): image width, padding offset; nxc = 16-pixel chunks per plane, ho = 1
};

constexpr int P_NA = 4, P_NRAW_B = 2, P_NDER = 2;

template <int RS, int DS, int KS>
size_t patch_param_smem(uint32_t a_slot) {
    return (size_t)RS * (a_slot + P_NRAW_B * HALF_BYTES * (KS / 2)) + (size_t)DS * P_NDER * HALF_BYTES * (KS / 2) + 1024 + 256;
}

// NCW converter warps (8 or 16): groups of four take the slabs in turn.
// PAIR: two CTAs of a cluster share every MMA (cta_group::2, 256 rows, each CTA stages half of the B rows), as in the
// Linear pair kernel. !PAIR: every CTA works alone on its 128 rows (cta_group::1) and stages all bn <= 64 B rows: no
// barrier or commit crosses an SM boundary.
// KS: 8-wide k steps per slab: 2 (16 pixels, delta tiles in the 64-byte swizzle) or 4 (32 pixels, 128-byte swizzle). Every
// slab costs about a thousand cycles of hand-offs and TMA row requests whatever it holds, so wide rows use 32 pixels.
template <int CH, int RS, int DS, int ACC, int NCW, bool PAIR, int KS>
__global__ void __launch_bounds__(32 * (3 + NCW), 1)
tagi_tc_conv_param_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmD0,
                          const __grid_constant__ CUtensorMap tmD1, const PatchParam pp, const int bn, int *status) {
    constexpr int NA = P_NA, NDER = P_NDER;
    constexpr int SK = KS * 8;                               // contraction steps (pixels) per slab
    constexpr uint32_t B_TILE = HALF_BYTES * (KS / 2);       // shared memory of one delta tile: up to 64 rows of SK floats
    constexpr uint32_t DER_SLOT = NDER * B_TILE;
    constexpr uint32_t NCOLS = 512;
    constexpr uint32_t acc_stride = ACC, A_COL0 = 2 * ACC;   // ACC >= bn: columns between the two accumulators
    static_assert(KS == 2 || KS == 4, "16 or 32 pixels per slab");
    static_assert(A_COL0 + DS * NA * SK <= 512, "tensor memory: accumulators + A slots");
    // columns of each accumulator a converter thread sums and stores: with accumulators of at most 64 columns the eight
    // converter warps split them 32 / 32, which leaves the registers to read a whole slab of patch values at once
    constexpr int NG = NCW / 4;                        // converter groups
    constexpr int SUMW = (ACC <= 64 ? 64 : 128) / NG;  // 64, 32 or 16
    static_assert(NCW == 8 || (NCW == 16 && ACC <= 64), "sixteen converter warps only with narrow accumulators");
    const uint32_t RAW_SLOT = pp.a_slot + P_NRAW_B * B_TILE;
    const uint32_t IDESC = make_idesc_tf32(PAIR ? 256 : 128, bn, 0, 0);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *aligned = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t raw_base = smem_base, der_base = smem_base + RS * RAW_SLOT;
    uint64_t *bars = reinterpret_cast<uint64_t *>(aligned + (size_t)RS * RAW_SLOT + (size_t)DS * DER_SLOT);
    constexpr int L = RS > DS ? RS : DS;
    uint64_t *raw_full = bars, *stage_done = bars + RS, *conv_done = bars + RS + L;
    uint64_t *acc_full = bars + RS + L + DS, *acc_empty = acc_full + 1;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta = PAIR ? cluster_ctarank() : 0;  // 0 issues the MMAs
    const int half = PAIR ? bn / 2 : bn;                          // B rows this CTA stages
    const int tile = PAIR ? blockIdx.y * 2 + (int)cta : blockIdx.y;  // this CTA's row tile: channels c0 .. c0 + CT - 1
    const int c0 = tile * pp.CT;
    const int col0 = (PAIR ? blockIdx.x >> 1 : blockIdx.x) * bn;  // the output channels of the tile
    const int brow0 = col0 + (int)cta * half;                     // this CTA's half of them (B rows)
    const uint32_t b_bytes = (uint32_t)half * SK * 4;             // a delta tile holds exactly the channel rows this CTA stages
    const int kb = (int)blockIdx.z * pp.slabs_per_slice;          // first slab of this slice
    const int nk = min(pp.total_slabs - kb, pp.slabs_per_slice);
    const int chunk_len = CH > 0 ? CH : nk;

    if (threadIdx.x == 0) {
        for (int s = 0; s < RS; s++) mbar_init(raw_full + s, 1);
        for (int s = 0; s < L; s++) mbar_init(stage_done + s, 2);            // one commit from each MMA issuer
        for (int s = 0; s < DS; s++) mbar_init(conv_done + s, PAIR ? 8 : 4);  // one warp group (of each CTA of a pair)
        mbar_init(acc_full, 2);
        mbar_init(acc_empty, PAIR ? 2 * NCW : NCW);                 // pairs: used in CTA 0 only
        *abort_flag = 0;
        mbar_init_fence();
        prefetch_tmap(&tmX);
        prefetch_tmap(&tmD0);
        prefetch_tmap(&tmD1);
    }
    if (warp == 1) {
        if (PAIR) tmem_alloc_pair(tmem_slot, NCOLS); else tmem_alloc(tmem_slot, NCOLS);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (PAIR) cluster_sync_all();  // the peer's barriers exist before anyone arrives on them
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (each CTA for itself)
        if (lane == 0) {
            for (int it = 0; it < nk; it++) {
                const int r = it % RS;
                if (it >= RS && !mbar_wait(stage_done + (it - RS) % L, ((it - RS) / L) & 1, abort_flag, status,
                                           ST_TIMEOUT_EMPTY))
                    break;
                const int t = kb + it;                 // slab -> (image, output row, chunk of the row); flat mode: ho = 1
                const int xc = t % pp.nxc, rr = t / pp.nxc, oy = rr % pp.ho, b = rr / pp.ho;
                mbar_arrive_expect_tx(raw_full + r, pp.a_bytes + P_NRAW_B * b_bytes);
                const uint32_t st = raw_base + r * RAW_SLOT;
                tma_load_4d(st, &tmX, xc * SK * pp.stride + pp.x0, oy * pp.stride + pp.y0, c0, b, raw_full + r);
                tma_load_4d(st + pp.a_slot, &tmD0, xc * SK, oy, brow0, b, raw_full + r);
                tma_load_4d(st + pp.a_slot + B_TILE, &tmD1, xc * SK, oy, brow0, b, raw_full + r);
            }
        }
    } else if (warp == 1 || warp == 2 + NCW) {
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
                    ok = PAIR ? mbar_wait_cluster(acc_empty, (c - 1) & 1, abort_flag, status, ST_TIMEOUT_ACC)
                              : mbar_wait(acc_empty, (c - 1) & 1, abort_flag, status, ST_TIMEOUT_ACC);
                    if (!ok) break;
                    f = 0;
                }
                ok = PAIR ? mbar_wait_cluster(conv_done + d, (it / DS) & 1, abort_flag, status, ST_TIMEOUT_CONV)
                          : mbar_wait(conv_done + d, (it / DS) & 1, abort_flag, status, ST_TIMEOUT_CONV);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t rb = raw_base + r * RAW_SLOT + pp.a_slot, ds = der_base + d * DER_SLOT;
                const uint32_t at = tmem + A_COL0 + d * (NA * SK);
                // K-major delta tiles: rows of SK floats, 8-row groups 8 * SK * 4 bytes apart, an 8-wide k step 32 bytes on
                constexpr uint32_t LBO = 16, KSTEP = 32 >> 4;
                constexpr uint32_t HI = desc_hi(KS == 2 ? 512 : 1024, KS == 2 ? SWZ_64B : SWZ_128B);
                const uint32_t rbl = desc_lo(rb, LBO), dsl = desc_lo(ds, LBO);
#pragma unroll
                for (int j = 0; j < KS; j++) {
                    const uint32_t fj = j == 0 ? f : 1u;
                    if (KS == 4) {
                        if (chain1) mma_kstep_cparam_w<PAIR, 1>(d1, d2, at + 8 * j, rbl + KSTEP * j, dsl + KSTEP * j, HI, IDESC, fj, fj);
                        else mma_kstep_cparam_w<PAIR, 2>(d1, d2, at + 8 * j, rbl + KSTEP * j, dsl + KSTEP * j, HI, IDESC, fj, fj);
                    } else if (PAIR) {
                        if (chain1) mma_kstep_cparam_pair<1>(d1, d2, at + 8 * j, rbl + KSTEP * j, dsl + KSTEP * j, HI, IDESC, fj, fj);
                        else mma_kstep_cparam_pair<2>(d1, d2, at + 8 * j, rbl + KSTEP * j, dsl + KSTEP * j, HI, IDESC, fj, fj);
                    } else {
                        if (chain1) mma_kstep_cparam_solo<1>(d1, d2, at + 8 * j, rbl + KSTEP * j, dsl + KSTEP * j, HI, IDESC, fj, fj);
                        else mma_kstep_cparam_solo<2>(d1, d2, at + 8 * j, rbl + KSTEP * j, dsl + KSTEP * j, HI, IDESC, fj, fj);
                    }
                }
                f = 1;
                // the raw slot may be refilled and the derived one overwritten (in both CTAs of a pair)
                if (PAIR) mma_commit_pair(stage_done + it % L); else mma_commit(stage_done + it % L);
                if (it % chunk_len == chunk_len - 1 || it == nk - 1) {
                    if (PAIR) mma_commit_pair(acc_full); else mma_commit(acc_full);
                }
            }
        }
    } else if (warp >= 2 && warp < 2 + NCW) {
        // ------------------------------------------------------------------ converters + accumulation + epilogue
        const int ct = threadIdx.x - 64;
        const int q = warp & 3;
        const int h = (warp - 2) >> 2;
        const int arow = q * 32 + lane;
        const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16);
        // this thread's row (channel cl of the tile, tap ky, kx): byte offset of its first value inside the patch.
        // Rows past the tile's CT * k * k read the patch's first values: finite numbers whose sums are never stored.
        const bool row_in_tile = arow < pp.CT * pp.k2;
        uint32_t row_off = 0;
        int flat_dx = 0;   // flat mode: this row's column shift
        {
            const int m = row_in_tile ? arow : 0;
            const int cl = m / pp.k2, tap = m - cl * pp.k2, ky = tap / pp.k, kx = tap - ky * pp.k;
            row_off = (uint32_t)(((cl * pp.k + ky) * pp.PW + kx + pp.lead) * 4);
            if (pp.flat) {   // one patch row per channel; `lead` is the halo
                row_off = (uint32_t)((cl * pp.PW + pp.lead + (ky - pp.off) * pp.W + (kx - pp.off)) * 4);
                flat_dx = kx - pp.off;
            }
        }
        const uint32_t step_b = (uint32_t)pp.stride * 4;
        float sum1[SUMW], sum2[SUMW];
#pragma unroll
        for (int i = 0; i < SUMW; i++) sum1[i] = sum2[i] = 0.f;

        auto drain = [&](int c) -> bool {
            if (!mbar_wait(acc_full, c & 1, abort_flag, status, ST_TIMEOUT_ACC)) return false;
            tc_fence_after_sync();
            if (SUMW >= 32) {
#pragma unroll
                for (int blk = 0; blk < SUMW / 32; blk++) {
                    float v[32];
                    tmem_ld_32x32(lane_addr + h * SUMW + blk * 32, v);
#pragma unroll
                    for (int i = 0; i < 32; i++) sum1[blk * 32 + i] += v[i];
                    tmem_ld_32x32(lane_addr + acc_stride + h * SUMW + blk * 32, v);
#pragma unroll
                    for (int i = 0; i < 32; i++) sum2[blk * 32 + i] += v[i];
                }
            } else {
                float v[16];
                tmem_ld_32x16(lane_addr + h * SUMW, v);
#pragma unroll
                for (int i = 0; i < 16; i++) sum1[i] += v[i];
                tmem_ld_32x16(lane_addr + acc_stride + h * SUMW, v);
#pragma unroll
                for (int i = 0; i < 16; i++) sum2[i] += v[i];
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (PAIR) mbar_arrive_cluster(acc_empty, 0); else mbar_arrive(acc_empty);
            }
            return true;
        };

        // two groups of four warps (h = 0 / 1) convert alternate slabs, as in the Linear pair kernel
        bool ok = true;
        int pending = -1, scanned = 0;
        auto note_chunk_ends = [&](int upto) {
            for (int sl = scanned; sl <= upto && sl < nk && ok; sl++)
                if (sl % chunk_len == chunk_len - 1 || sl == nk - 1) {
                    if (pending >= 0) ok = drain(pending);
                    pending = sl / chunk_len;
                }
            scanned = upto + 1;
        };
        const int gt = ct & 127;  // thread index inside the group
        for (int it = h; it < nk && ok; it += NG) {
            const int r = it % RS, d = it % DS;
            ok = mbar_wait(raw_full + r, (it / RS) & 1, abort_flag, status, ST_TIMEOUT_RAW) &&
                 (it < DS || mbar_wait(stage_done + (it - DS) % L, ((it - DS) / L) & 1, abort_flag, status,
                                       ST_TIMEOUT_EMPTY));
            if (!ok) break;
            const uint32_t rs = raw_base + r * RAW_SLOT, rb = rs + pp.a_slot, ds = der_base + d * DER_SLOT;

            constexpr int KW = (SUMW == 32 && NCW == 8) ? 16 : 8;   // pixels read before they are converted
#pragma unroll
            for (int kh = 0; kh < SK / KW; kh++) {
                float x[KW];
#pragma unroll
                for (int i = 0; i < KW; i++)
                    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(x[i]) : "r"(rs + row_off + (kh * KW + i) * step_b));
                if (pp.flat && flat_dx != 0) {
                    // column of pixel i of the slab: (p0 + i) mod W; a tap that leaves the image row reads padding
                    int px = ((kb + it) % pp.nxc * SK + kh * KW) % pp.W;
#pragma unroll
                    for (int i = 0; i < KW; i++) {
                        if ((unsigned)(px + flat_dx) >= (unsigned)pp.W) x[i] = 0.f;
                        px = px + 1 == pp.W ? 0 : px + 1;
                    }
                }
#pragma unroll
                for (int p8 = 0; p8 < KW / 8; p8++) {
                    const uint32_t at = lane_addr + A_COL0 + d * (NA * SK) + kh * KW + p8 * 8;
                    float t0[8], t1[8], qq[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const float v = x[p8 * 8 + i];
                        qq[i] = v * v, t0[i] = hi_part(v), t1[i] = hi_part(qq[i]);
                    }
                    tmem_st_32x8(at + 0 * SK, t0);
                    tmem_st_32x8(at + 1 * SK, t1);
#pragma unroll
                    for (int i = 0; i < 8; i++) t0[i] = x[p8 * 8 + i] - t0[i], t1[i] = qq[i] - t1[i];
                    tmem_st_32x8(at + 2 * SK, t0);
                    tmem_st_32x8(at + 3 * SK, t1);
                }
            }
            // the delta tiles (dmu_z, dvar_z, the channel rows this CTA stages): lo parts at the same swizzled offsets
#pragma unroll
            for (int c = 0; c < (int)(B_TILE / 2048); c++) {
                const uint32_t o = gt * 16 + c * 2048;
                if (o >= b_bytes) break;
                const float4 b0 = lds128(rb + o), b1 = lds128(rb + B_TILE + o);
                sts128(ds + 0 * B_TILE + o, lo_part(b0));
                sts128(ds + 1 * B_TILE + o, lo_part(b1));
            }
            fence_proxy_async_smem();
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (PAIR) mbar_arrive_cluster(conv_done + d, 0); else mbar_arrive(conv_done + d);
            }
            if (pending >= 0) {
                ok = drain(pending);
                pending = -1;
            }
            note_chunk_ends(it + NG - 1);
        }
        if (ok) note_chunk_ends(nk - 1);
        if (ok && pending >= 0) ok = drain(pending);

        // epilogue: row (c, tap) of the tile is weight column kc = c0 * k2 + arow; this thread holds 64 output channels
        // of it. out[co][kc]: for one co the 32 lanes of a warp write 32 consecutive kc (coalesced).
        const int kc = c0 * pp.k2 + arow;
        if (ok && row_in_tile && kc < pp.Kc && h * SUMW < bn) {
            float *o1 = pp.out1 + (long)blockIdx.z * pp.slice_elems + kc;
            float *o2 = pp.out2 + (long)blockIdx.z * pp.slice_elems + kc;
            const int cbase = col0 + h * SUMW, valid = min(bn - h * SUMW, pp.fo - cbase);
#pragma unroll
            for (int i0 = 0; i0 < SUMW; i0 += 8) {
                float sc[8];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    sc[u] = 1.f;
                    if (pp.scale && i0 + u < valid) sc[u] = __ldg(pp.scale + (long)(cbase + i0 + u) * pp.Kc + kc);
                }
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    if (i0 + u >= valid) continue;
                    const long idx = (long)(cbase + i0 + u) * pp.Kc;
                    o1[idx] = sum1[i0 + u] * sc[u];
                    o2[idx] = sum2[i0 + u] * sc[u] * sc[u];
                }
            }
        }
    }
    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    if (PAIR) cluster_sync_all();  // neither CTA leaves (or frees tensor memory) while the other may still signal or read it
    if (warp == 1) {
        if (*abort_flag) {
            const long long t0 = clock64();
            while (clock64() - t0 < 4000000LL) {
            }
        }
        if (PAIR) tmem_dealloc_pair(tmem, NCOLS); else tmem_dealloc(tmem, NCOLS);
    }
}

// Sum of the contraction slices in slice order, then the scaling by var_w and var_w^2
__global__ void __launch_bounds__(256) patch_reduce_slices_kernel(const float *__restrict__ part1,
                                                                  const float *__restrict__ part2,
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

// =====================================================================================================
// Forward pass and stride-1 state pass as implicit GEMMs with TMA-loaded patches.
//
//   forward   rows = output pixels, columns = output channels, contraction over (tap, input channel):
//             A(pixel (b, oy, ox); tap (ky, kx), ci) = mu_a / var_a [b][ci][oy - off + ky][ox - off + kx]
//             B = the weights regrouped as [co][tap][ci] (K-major)
//   state     rows = input pixels, columns = input channels, contraction over (tap, output channel):
//             A(pixel (b, y, x); tap, co) = dmu_z / dvar_z [b][co][y + off - ky][x + off - kx]
//             B = mu_w regrouped as [(tap, co)][ci] (MN-major)
// A CTA's 128 rows are NI images x TR image rows x GW columns of the pixel grid (TR * GW <= 128; several whole images
// per tile when an image has at most 64 pixels). One k-slab is 16 channels of one tap; the contraction runs channel
// block by channel block, and inside a block over its k*k taps. The A operand of all k*k slabs of a channel block is ONE
// box of the source tensor per operand, [PW columns][TR + k - 1 rows][16 channels][NI images], loaded once into a ring of
// its own (two blocks deep) and read k*k times with the tap's shift: a tap moves the converter thread's read position by
// (ky, kx) inside the patch. A TMA box must start on a 16-byte boundary, so the box always starts at the same aligned
// column and is a few columns wider than the image. Zeros arrive for coordinates outside the image: the padding rule
// without masks. Loading per tap instead cost 4.5 times the shared-memory fill traffic and left the kernel bound by the
// L2's bandwidth. The converter thread of pixel (py, px) reads its 16 channel values at (c, py + ky, px + kx) and writes
// the TF32 hi / lo (and mu^2 + var) operands to tensor memory; everything downstream (B-side conversion, MMAs, chunked
// accumulation, barriers) is the Linear pair kernel's.
// =====================================================================================================
struct PixParam {
    // pixel grid of the rows (output grid for the forward pass, input grid for the state pass) and tiling
    int GH, GW, TR, NI, tiles_y, tiles_total, B;
    // source tensor patches
    int k, k2, cblocks;        // taps per side, taps, 16-channel blocks of the contraction (source channels / 16)
    int sign, off;             // +1: source pixel = p - off + tap (forward); -1: p + off - tap (state)
    int PW, PR, lead;          // patch row pitch in floats, rows per channel (TR + k - 1); `lead`: column of grid x = 0
                               // for the smallest tap shift
    int x0, y0;                // coordinates of the patch's first column (multiple of 4, may be negative) and of its
                               // first row relative to the tile's first grid row
    uint32_t a_bytes, a_slot;  // bytes of one operand's patch box; ring slot reserved for it (multiple of 1024)
    int RS, AS;                // depth of the B ring and of the patch ring
    // epilogue
    float *out1, *out2, *out3; // [B][cols][GH*GW]; out3: ReLU Jacobian (forward with RELU)
    const float *aux1, *aux2;  // forward: bias vectors (may be null); state: aux1 = Jacobian [B][cols][GH*GW] (may be null)
    int cols;                  // output channels (forward) / input channels (state)
};

constexpr int PIX_MAX_RS = 8, PIX_MAX_AS = 3;
constexpr int PIX_MAX_SLABS = 768, PIX_TAB_BYTES = PIX_MAX_SLABS * 8;   // slab table: k*k taps x 16-channel blocks

template <int OP>
size_t pix_smem(uint32_t a_slot, int AS, int RS, int DS) {
    return (size_t)AS * 2 * a_slot + (size_t)RS * PairTraits<OP>::NRAW_B * HALF_BYTES +
           (size_t)DS * PairTraits<OP>::NDER * HALF_BYTES + 1024 + 256 + PIX_TAB_BYTES;
}

// ACC: tensor-memory columns between the two accumulators (>= bn); DS derived slots
// NCW converter warps (8 or 16): groups of four take the slabs in turn
template <int OP, int CH, int DS, int ACC, bool RELU, int NCW>
__global__ void __launch_bounds__(32 * (3 + NCW), 1)
tagi_tc_conv_pix_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
                        const __grid_constant__ CUtensorMap tmB0, const __grid_constant__ CUtensorMap tmB1,
                        const PixParam pp, const int bn, int *status) {
    using T = OpTraits<OP>;
    using S = PairTraits<OP>;
    constexpr int NRAW_B = S::NRAW_B, NDER = S::NDER, NA = S::NA;
    constexpr uint32_t DER_SLOT = NDER * HALF_BYTES;
    constexpr uint32_t NCOLS = 512;
    constexpr uint32_t acc_stride = ACC, A_COL0 = 2 * ACC;
    static_assert(A_COL0 + DS * NA * BK <= 512, "tensor memory: accumulators + A slots");
    // columns of each accumulator a converter thread sums and stores: with accumulators of at most 64 columns the eight
    // converter warps split them 32 / 32, which leaves the registers to read a whole slab of A values at once
    constexpr int NG = NCW / 4;                        // converter groups
    constexpr int SUMW = (ACC <= 64 ? 64 : 128) / NG;  // 64, 32 or 16
    static_assert(NCW == 8 || NCW == 16, "eight or sixteen converter warps");
    const int RS = pp.RS, AS = pp.AS;
    constexpr uint32_t RAW_SLOT = NRAW_B * HALF_BYTES;               // B ring slot: the raw B half tiles of one slab
    const uint32_t A_SLOT = 2 * pp.a_slot;                           // patch ring slot: both operands of a channel block
    const uint32_t IDESC = make_idesc_tf32(256, bn, 0, T::B_MN);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *aligned = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t patch_base = smem_base, raw_base = patch_base + AS * A_SLOT, der_base = raw_base + RS * RAW_SLOT;
    uint64_t *bars = reinterpret_cast<uint64_t *>(aligned + (size_t)AS * A_SLOT + (size_t)RS * RAW_SLOT + (size_t)DS * DER_SLOT);
    constexpr int LMAX = PIX_MAX_RS > DS ? PIX_MAX_RS : DS;
    const int L = RS > DS ? RS : DS;
    uint64_t *raw_full = bars, *stage_done = bars + PIX_MAX_RS, *conv_done = stage_done + LMAX;
    uint64_t *acc_full = conv_done + DS, *acc_empty = acc_full + 1;
    uint64_t *a_full = acc_empty + 1, *a_free = a_full + PIX_MAX_AS;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(a_free + PIX_MAX_AS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    // per slab: byte offset of the slab's read position inside the patch ring (ring slot + tap shift), and its channel block
    uint2 *slab_tab = reinterpret_cast<uint2 *>(bars + 32);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta = cluster_ctarank();
    const int half = bn / 2;
    const int tile = blockIdx.y * 2 + (int)cta;                    // this CTA's pixel tile
    const int bt = tile / pp.tiles_y, ytile = tile - bt * pp.tiles_y;
    const int b0 = bt * pp.NI, py0 = ytile * pp.TR;                // first image and first grid row of the tile
    const int col0 = (blockIdx.x >> 1) * bn;
    const int brow0 = col0 + (int)cta * half;
    const int nk = pp.k2 * pp.cblocks;
    const int chunk_len = CH > 0 ? CH : nk;
    for (int i = threadIdx.x; i < nk; i += blockDim.x) {
        const int cb = i / pp.k2, tap = i - cb * pp.k2, ky = tap / pp.k, kx = tap - ky * pp.k;
        const int sy = pp.sign > 0 ? ky : pp.k - 1 - ky, sx = pp.sign > 0 ? kx : pp.k - 1 - kx;
        slab_tab[i] = make_uint2((uint32_t)(cb % pp.AS) * 2 * pp.a_slot + (uint32_t)((sy * pp.PW + sx) * 4), (uint32_t)cb);
    }
    // a B tile holds this CTA's half of the columns: K-major bn / 2 rows of 64 bytes, MN-major 2 KiB boxes of 32 rows
    const int b_boxes = (half + 31) / 32;
    const uint32_t b_bytes = T::B_MN ? (uint32_t)b_boxes * 2048 : (uint32_t)half * 64;

    if (threadIdx.x == 0) {
        for (int s = 0; s < RS; s++) mbar_init(raw_full + s, 1);
        for (int s = 0; s < L; s++) mbar_init(stage_done + s, 2);
        for (int s = 0; s < DS; s++) mbar_init(conv_done + s, NCONV_WARPS);
        for (int s = 0; s < AS; s++) {
            mbar_init(a_full + s, 1);
            mbar_init(a_free + s, NCW);   // every converter warp of this CTA releases a patch once
        }
        mbar_init(acc_full, 2);
        mbar_init(acc_empty, 2 * NCW);
        *abort_flag = 0;
        mbar_init_fence();
        prefetch_tmap(&tmA0);
        prefetch_tmap(&tmA1);
        prefetch_tmap(&tmB0);
        if (OP == OP_FWD) prefetch_tmap(&tmB1);
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot, NCOLS);
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (each CTA for itself)
        if (lane == 0) {
            int tap = 0, cb = 0;   // slab it = cb * k2 + tap
            for (int it = 0; it < nk; it++) {
                if (tap == 0) {
                    // the patch of channel block cb: both operands, once for all its taps
                    const int a = cb % AS;
                    if (cb >= AS && !mbar_wait(a_free + a, ((cb / AS) - 1) & 1, abort_flag, status, ST_TIMEOUT_EMPTY)) break;
                    mbar_arrive_expect_tx(a_full + a, 2 * pp.a_bytes);
                    const uint32_t pa = patch_base + a * A_SLOT;
                    tma_load_4d(pa, &tmA0, pp.x0, py0 + pp.y0, cb * 16, b0, a_full + a);
                    tma_load_4d(pa + pp.a_slot, &tmA1, pp.x0, py0 + pp.y0, cb * 16, b0, a_full + a);
                }
                const int r = it % RS;
                if (it >= RS && !mbar_wait(stage_done + (it - RS) % L, ((it - RS) / L) & 1, abort_flag, status,
                                           ST_TIMEOUT_EMPTY))
                    break;
                mbar_arrive_expect_tx(raw_full + r, NRAW_B * b_bytes);
                const uint32_t st = raw_base + r * RAW_SLOT;
                const int k0 = it * BK;
                if (T::B_MN) {
                    for (int gb = 0; gb < b_boxes; gb++)
                        tma_load_2d(st + gb * 2048, &tmB0, brow0 + 32 * gb, k0, raw_full + r);
                } else {
                    tma_load_2d(st, &tmB0, k0, brow0, raw_full + r);
                    if (OP == OP_FWD) tma_load_2d(st + HALF_BYTES, &tmB1, k0, brow0, raw_full + r);
                }
                if (++tap == pp.k2) tap = 0, cb++;
            }
        }
    } else if (warp == 1 || warp == 2 + NCW) {
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
                const uint32_t rb = raw_base + r * RAW_SLOT, ds = der_base + d * DER_SLOT;
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
                mma_commit_pair(stage_done + it % L);
                if (it % chunk_len == chunk_len - 1 || it == nk - 1) mma_commit_pair(acc_full);
            }
        }
    } else if (warp >= 2 && warp < 2 + NCW) {
        // ------------------------------------------------------------------ converters + accumulation + epilogue
        const int ct = threadIdx.x - 64;
        const int q = warp & 3;
        const int h = (warp - 2) >> 2;
        const int arow = q * 32 + lane;
        const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16);
        // this thread's pixel: image il of the tile, grid row pyl, grid column px
        const int per_img = pp.TR * pp.GW;
        const bool row_in_tile = arow < pp.NI * per_img;
        const int mm = row_in_tile ? arow : 0;
        const int il = mm / per_img, rem = mm - il * per_img, pyl = rem / pp.GW, px = rem - pyl * pp.GW;
        // byte offset of (channel 0, patch row pyl, column px + lead) of image il inside a patch; a channel is cstride on
        const uint32_t cstride = (uint32_t)(pp.PR * pp.PW * 4);
        const uint32_t row_off = (uint32_t)(((il * 16 * pp.PR + pyl) * pp.PW + px + pp.lead) * 4);
        int released = 0;   // channel blocks whose patch this warp has released
        float sum1[SUMW], sum2[SUMW];
#pragma unroll
        for (int i = 0; i < SUMW; i++) sum1[i] = sum2[i] = 0.f;

        auto drain = [&](int c) -> bool {
            if (!mbar_wait(acc_full, c & 1, abort_flag, status, ST_TIMEOUT_ACC)) return false;
            tc_fence_after_sync();
            if (SUMW >= 32) {
#pragma unroll
                for (int blk = 0; blk < SUMW / 32; blk++) {
                    float v[32];
                    tmem_ld_32x32(lane_addr + h * SUMW + blk * 32, v);
#pragma unroll
                    for (int i = 0; i < 32; i++) sum1[blk * 32 + i] += v[i];
                    tmem_ld_32x32(lane_addr + acc_stride + h * SUMW + blk * 32, v);
#pragma unroll
                    for (int i = 0; i < 32; i++) sum2[blk * 32 + i] += v[i];
                }
            } else {
                float v[16];
                tmem_ld_32x16(lane_addr + h * SUMW, v);
#pragma unroll
                for (int i = 0; i < 16; i++) sum1[i] += v[i];
                tmem_ld_32x16(lane_addr + acc_stride + h * SUMW, v);
#pragma unroll
                for (int i = 0; i < 16; i++) sum2[i] += v[i];
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty, 0);
            return true;
        };

        bool ok = true;
        int pending = -1, scanned = 0;
        auto note_chunk_ends = [&](int upto) {
            for (int sl = scanned; sl <= upto && sl < nk && ok; sl++)
                if (sl % chunk_len == chunk_len - 1 || sl == nk - 1) {
                    if (pending >= 0) ok = drain(pending);
                    pending = sl / chunk_len;
                }
            scanned = upto + 1;
        };
        const int gt = ct & 127;
        for (int it = h; it < nk && ok; it += NG) {
            const int r = it % RS, d = it % DS;
            ok = mbar_wait(raw_full + r, (it / RS) & 1, abort_flag, status, ST_TIMEOUT_RAW) &&
                 (it < DS || mbar_wait(stage_done + (it - DS) % L, ((it - DS) / L) & 1, abort_flag, status,
                                       ST_TIMEOUT_EMPTY));
            if (!ok) break;
            const uint32_t rb = raw_base + r * RAW_SLOT, ds = der_base + d * DER_SLOT;
            // slab = (channel block cb, tap): the tap moves this thread's read position inside the block's patch
            const uint2 te = slab_tab[it];
            const int cb = (int)te.y;
            ok = mbar_wait(a_full + cb % AS, (cb / AS) & 1, abort_flag, status, ST_TIMEOUT_RAW);
            if (!ok) break;
            const uint32_t src = patch_base + row_off + te.x;

            constexpr int KW = (SUMW == 32 && NCW == 8) ? 16 : 8;   // channels read before they are converted
#pragma unroll
            for (int kh = 0; kh < 16 / KW; kh++) {
                float a0[KW], a1[KW];
#pragma unroll
                for (int i = 0; i < KW; i++) {
                    const uint32_t o = src + (kh * KW + i) * cstride;
                    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(a0[i]) : "r"(o));
                    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(a1[i]) : "r"(o + pp.a_slot));
                }
#pragma unroll
                for (int p8 = 0; p8 < KW / 8; p8++) {
                    const uint32_t at = lane_addr + A_COL0 + d * (NA * BK) + kh * KW + p8 * 8;
                    float t0[8], t1[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) t0[i] = hi_part(a0[p8 * 8 + i]), t1[i] = hi_part(a1[p8 * 8 + i]);
                    tmem_st_32x8(at + 0 * BK, t0);
                    tmem_st_32x8(at + 1 * BK, t1);
#pragma unroll
                    for (int i = 0; i < 8; i++) t0[i] = a0[p8 * 8 + i] - t0[i], t1[i] = a1[p8 * 8 + i] - t1[i];
                    tmem_st_32x8(at + 2 * BK, t0);
                    tmem_st_32x8(at + 3 * BK, t1);
                    if (OP == OP_FWD) {
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            const float sq = fmaf(a0[p8 * 8 + i], a0[p8 * 8 + i], a1[p8 * 8 + i]);
                            t0[i] = hi_part(sq);
                            t1[i] = sq - t0[i];
                        }
                        tmem_st_32x8(at + 4 * BK, t0);
                        tmem_st_32x8(at + 5 * BK, t1);
                    }
                }
            }
            {
                // This warp's next slab is it + NG: the patches of all blocks below that slab's block are no longer
                // read by it (its slabs come in increasing order), whether or not it had a slab in them.
                const int nb = min((it + NG) / pp.k2, pp.cblocks);
                __syncwarp();
                for (; released < nb; released++)
                    if (lane == 0) mbar_arrive(a_free + released % AS);
            }
            // B halves: two 16-byte chunks per thread of the group
#pragma unroll
            for (int c = 0; c < 2; c++) {
                const uint32_t o = gt * 16 + c * (HALF_BYTES / 2);
                if (o >= b_bytes) break;
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
            note_chunk_ends(it + NG - 1);
        }
        if (ok) note_chunk_ends(nk - 1);
        if (ok && pending >= 0) ok = drain(pending);
        // (patches still unreleased here belong to the last blocks: nobody waits for them)

        // epilogue: [image][channel][pixel]; the 32 lanes of a warp hold consecutive pixels, so each channel's store is
        // (mostly) one contiguous run
        const int b = b0 + il, py = py0 + pyl;
        if (ok && row_in_tile && b < pp.B && py < pp.GH && h * SUMW < bn) {
            const long npix = (long)pp.GH * pp.GW;
            const long base = (long)b * pp.cols * npix + (long)py * pp.GW + px;
            const int cbase = col0 + h * SUMW, valid = min(bn - h * SUMW, pp.cols - cbase);
#pragma unroll
            for (int i0 = 0; i0 < SUMW; i0 += 8) {
                float sc[8];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    sc[u] = 1.f;
                    if (OP != OP_FWD && pp.aux1 && i0 + u < valid) sc[u] = __ldg(pp.aux1 + base + (long)(cbase + i0 + u) * npix);
                }
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    if (i0 + u >= valid) continue;
                    const int col = cbase + i0 + u;
                    const long idx = base + (long)col * npix;
                    float o1 = sum1[i0 + u], o2 = sum2[i0 + u];
                    if (OP == OP_FWD) {
                        if (pp.aux1) {
                            o1 += __ldg(pp.aux1 + col);
                            o2 += __ldg(pp.aux2 + col);
                        }
                    } else {
                        o1 *= sc[u];
                        o2 = o2 * sc[u] * sc[u];
                    }
                    if (RELU) __stcs(pp.out3 + idx, relu_moments(o1, o2));
                    __stcs(pp.out1 + idx, o1);
                    __stcs(pp.out2 + idx, o2);
                }
            }
        }
    }
    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        if (*abort_flag) {
            const long long t0 = clock64();
            while (clock64() - t0 < 4000000LL) {
            }
        }
        tmem_dealloc_pair(tmem, NCOLS);
    }
}

// 4-D tensor map over a [B][C][H][W] FP32 tensor
int make_tmap_nchw(CUtensorMap *tm, const float *ptr, int W, int H, int C, int B, unsigned bx, unsigned by, unsigned bc,
                   CUtensorMapSwizzle swz, unsigned bb = 1) {
    EncodeTiledFn fn = tc_encode_fn();
    if (!fn) return fail(TAGI_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[4] = {(cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)C, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)W * 4, (cuuint64_t)W * H * 4, (cuuint64_t)W * H * C * 4};
    cuuint32_t box[4] = {bx, by, bc, bb};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(TAGI_ERR_CUDA, "cuTensorMapEncodeTiled (4-D) failed with code " + std::to_string((int)r));
    return TAGI_OK;
}

struct ParamPlan {
    PatchParam pp;
    int bn, col_tiles, row_pairs, row_tiles, slices, sk;   // sk: pixels per slab (16 or 32)
    bool pair;   // CTA pairs (tiles wider than 64 columns) or single CTAs
};

inline int round_up4(int v) { return (v + 3) & ~3; }

bool plan_param(const tagi_conv2d_geom &g, ParamPlan *out) {
    const int off = g.pad_type == 1 ? g.pad : 0;
    const int k2 = g.k * g.k;
    if (k2 > 128 || g.fo < 16) return false;
    PatchParam &p = out->pp;
    // flat mode: rows are not 16-byte multiples but planes are, and the layer keeps the image size at stride 1
    const bool flat = (g.wi % 4 || g.wo % 4) && g.stride == 1 && g.wi == g.wo && g.hi == g.ho && (g.hi * g.wi) % 4 == 0;
    if ((g.wi % 4 || g.wo % 4) && !flat) return false;
    p.flat = flat ? 1 : 0, p.W = g.wi, p.off = off;
    p.fi = g.fi, p.k = g.k, p.k2 = k2, p.Kc = k2 * g.fi, p.fo = g.fo;
    p.CT = 128 / k2 < g.fi ? 128 / k2 : g.fi;
    // output channels per tile: one tile when it fits, else the width that wastes least
    int bn = g.fo <= 128 ? ((g.fo + 15) / 16) * 16 : 128;
    if (g.fo > 128) {
        long best = -1;
        for (int w = 128; w >= 64; w -= 16) {
            const long waste = (long)((g.fo + w - 1) / w) * w - g.fo;
            if (best < 0 || waste < best) best = waste, bn = w;
        }
    }
    static const int solo_mode = [] { const char *v = getenv("TAGI_B200_CONV_SOLO"); return v ? atoi(v) : 1; }();
    out->pair = bn > 64 || solo_mode == 0;
    // 32 pixels per slab for single-CTA tiles (measured: 20 % faster on the 64-channel ResNet layers, nothing or a loss
    // on CTA pairs, whose tensor memory holds only two slots of that size), unless the row's last chunk would be mostly
    // padding
    const int pad16 = (g.wo + 15) / 16 * 16, pad32 = (g.wo + 31) / 32 * 32;
    static const int force_sk = [] { const char *v = getenv("TAGI_B200_CONV_SLABK"); return v ? atoi(v) : 0; }();
    const int sk = force_sk == 16 || force_sk == 32 ? force_sk : (!out->pair && pad32 * 85 <= pad16 * 100 ? 32 : 16);
    out->sk = flat ? 16 : sk;
    p.ho = g.ho, p.nxc = (g.wo + sk - 1) / sk;
    p.stride = g.stride;
    p.lead = round_up4(off) - off;
    p.x0 = -round_up4(off), p.y0 = -off;
    p.PW = round_up4((sk - 1) * g.stride + g.k + p.lead);
    if (flat) {
        // one row per channel: [p0 - halo, p0 + 16 + halo), halo = the largest tap shift off * W + off rounded up to 16 bytes
        const int halo = round_up4(off * g.wi + off);
        p.ho = 1, p.nxc = (g.hi * g.wi + 15) / 16;
        p.lead = halo, p.x0 = -halo, p.y0 = 0;
        p.PW = 16 + 2 * halo;
        if (g.k - 1 - off > off) return false;   // (taps reach further down-right than up-left: not a same-size layer)
    }
    // The 32 lanes of a converter warp read 32 consecutive (channel, ky, kx) rows of the patch, i.e. about 11 patch rows of
    // k consecutive floats each. With a pitch that is a multiple of 32 bytes those rows fall on 4 bank groups (measured:
    // half of the LSU's shared-memory wavefronts were conflict replays with a pitch of 40 floats); an odd multiple of 16
    // bytes spreads them over 8.
    if ((p.PW / 4) % 2 == 0) p.PW += 4;
    if (p.PW > 256 || p.CT > 256 || g.k > 256) return false;
    p.a_bytes = (uint32_t)p.PW * (flat ? 1 : g.k) * p.CT * 4;
    p.a_slot = (p.a_bytes + 1023u) & ~1023u;
    if (p.a_slot > 24 * 1024) return false;
    const long total = (long)g.B * p.ho * p.nxc;
    if (total >= (1L << 31)) return false;
    p.total_slabs = (int)total;
    out->bn = bn;
    out->col_tiles = (g.fo + bn - 1) / bn;
    const int row_tiles = (g.fi + p.CT - 1) / p.CT;
    out->row_tiles = row_tiles;
    out->row_pairs = (row_tiles + 1) / 2;
    // slices: about one wave of CTAs (or CTA pairs), at least 32 slabs each
    const long pairs = out->pair ? (long)out->row_pairs * out->col_tiles : (long)row_tiles * out->col_tiles;
    const int slots = out->pair ? tc_sm_budget() / 2 : tc_sm_budget();
    long s = pairs >= slots ? 1 : slots / pairs;
    if (s > total / 32) s = total / 32;
    if (s < 1) s = 1;
    p.slabs_per_slice = (int)((total + s - 1) / s);
    out->slices = (int)((total + p.slabs_per_slice - 1) / p.slabs_per_slice);
    return true;
}

// 2-D tensor map over a row-major FP32 matrix [outer][inner] (the regrouped weights): K-major half tiles are boxes of
// 16 x 64 in the 64-byte swizzle, MN-major ones boxes of 32 x 16 in the 128-byte swizzle with 32-byte atoms
int make_tmap_weights(CUtensorMap *tm, const float *ptr, uint64_t inner, uint64_t outer, bool mn_major, unsigned rows = 64) {
    EncodeTiledFn fn = tc_encode_fn();
    if (!fn) return fail(TAGI_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {inner * sizeof(float)};
    cuuint32_t box[2] = {mn_major ? 32u : (cuuint32_t)BK, mn_major ? (cuuint32_t)BK : (cuuint32_t)rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE,
                    mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_64B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(TAGI_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
    return TAGI_OK;
}

// The contraction index of the patch kernels is (channel block cb, tap, channel cl inside the block), ci = cb*16 + cl.
// forward: w2[co][(cb * k2 + tap) * 16 + cl] = w[co][ci * k2 + tap] for the means and the variances
__global__ void __launch_bounds__(256) regroup_weights_fwd_kernel(const float *__restrict__ w0, const float *__restrict__ w1,
                                                                  int fo, int fi, int k2, float *__restrict__ o0,
                                                                  float *__restrict__ o1) {
    const long total = (long)fo * fi * k2;
    const int cblocks = fi / 16;
    for (long t = (long)blockIdx.x * 256 + threadIdx.x; t < total; t += (long)gridDim.x * 256) {
        const int cl = (int)(t & 15);
        long r = t >> 4;
        const int tap = (int)(r % k2);
        r /= k2;
        const int cb = (int)(r % cblocks), co = (int)(r / cblocks);
        const long src = ((long)co * fi + cb * 16 + cl) * k2 + tap;
        o0[t] = __ldg(w0 + src);
        o1[t] = __ldg(w1 + src);
    }
}
// state pass (contraction over output channels co = cb*16 + cl): w2[(cb * k2 + tap) * 16 + cl][ci] = w[co][ci * k2 + tap]
__global__ void __launch_bounds__(256) regroup_weights_state_kernel(const float *__restrict__ w, int fo, int fi, int k2,
                                                                    float *__restrict__ o) {
    const long total = (long)fo * fi * k2;
    for (long t = (long)blockIdx.x * 256 + threadIdx.x; t < total; t += (long)gridDim.x * 256) {
        const int ci = (int)(t % fi);
        long r = t / fi;
        const int cl = (int)(r & 15);
        r >>= 4;
        const int tap = (int)(r % k2), cb = (int)(r / k2);
        o[t] = __ldg(w + ((long)(cb * 16 + cl) * fi + ci) * k2 + tap);
    }
}

struct PixPlan {
    PixParam pp;
    int bn, col_tiles, row_pairs, src_C, src_H, src_W;
};

inline int floor4(int v) { return v >= 0 ? v & ~3 : -(((-v) + 3) & ~3); }

// pass: CONV_PASS_FWD or CONV_PASS_STATE
bool plan_pix(const tagi_conv2d_geom &g, int pass, PixPlan *out) {
    if (g.stride != 1) return false;
    const int off = g.pad_type == 1 ? g.pad : 0;
    const bool fwd = pass == CONV_PASS_FWD;
    PixParam &p = out->pp;
    p.GH = fwd ? g.ho : g.hi, p.GW = fwd ? g.wo : g.wi, p.B = g.B;
    out->src_C = fwd ? g.fi : g.fo, out->src_H = fwd ? g.hi : g.ho, out->src_W = fwd ? g.wi : g.wo;
    p.cols = fwd ? g.fo : g.fi;
    if (out->src_C % 16 || out->src_W % 4 || p.GW > 128 || p.cols < 16 || p.cols % 4) return false;
    p.k = g.k, p.k2 = g.k * g.k, p.cblocks = out->src_C / 16;
    if ((long)p.k2 * p.cblocks > PIX_MAX_SLABS) return false;
    p.sign = fwd ? +1 : -1, p.off = off;
    if (p.GH * p.GW <= 64) {
        p.NI = 128 / (p.GH * p.GW), p.TR = p.GH;
    } else {
        p.NI = 1, p.TR = 128 / p.GW < p.GH ? 128 / p.GW : p.GH;
    }
    if (p.NI > g.B) p.NI = g.B;
    p.tiles_y = (p.GH + p.TR - 1) / p.TR;
    p.tiles_total = ((g.B + p.NI - 1) / p.NI) * p.tiles_y;
    // x shift of a tap: forward kx - off, state off - kx; the box starts at the smallest shift rounded down to 16 bytes
    const int dxmin = fwd ? -off : off - (g.k - 1);
    p.x0 = floor4(dxmin);
    p.lead = dxmin - p.x0;
    p.PW = (p.GW - 1 + g.k - 1 + p.lead + 1 + 3) & ~3;
    p.PR = p.TR + g.k - 1;
    p.y0 = dxmin;   // the smallest tap shift is the same in y
    if (p.PW > 256 || p.PR > 256) return false;
    p.a_bytes = (uint32_t)p.PW * p.PR * 16 * p.NI * 4;
    p.a_slot = (p.a_bytes + 1023u) & ~1023u;
    if (p.a_slot > 24 * 1024) return false;
    int bn = p.cols <= 128 ? ((p.cols + 15) / 16) * 16 : 128;
    if (p.cols > 128) {
        long best = -1;
        for (int w = 128; w >= 64; w -= 16) {
            const long waste = (long)((p.cols + w - 1) / w) * w - p.cols;
            if (best < 0 || waste < best) best = waste, bn = w;
        }
    }
    out->bn = bn;
    out->col_tiles = (p.cols + bn - 1) / bn;
    out->row_pairs = (p.tiles_total + 1) / 2;
    return true;
}

template <int OP, int DS, int ACC, int NCW>
int launch_pix(const CUtensorMap &a0, const CUtensorMap &a1, const CUtensorMap &b0, const CUtensorMap &b1, PixPlan &plan,
               bool relu, cudaStream_t st) {
    int *status = tc_status_word();
    if (!status) return fail(TAGI_ERR_CUDA, "cannot allocate the tensor-core status word");
    PixParam &p = plan.pp;
    // rings: two patch slots (three when they are small), then as many B slots as fit beside the derived ring
    const size_t budget = 227 * 1024 - 1280 - PIX_TAB_BYTES;
    const size_t der = (size_t)DS * PairTraits<OP>::NDER * HALF_BYTES;
    const size_t raw = (size_t)PairTraits<OP>::NRAW_B * HALF_BYTES;
    p.AS = 2 * (size_t)p.a_slot * 3 + der + 4 * raw <= budget ? 3 : 2;
    long rs = ((long)budget - (long)der - (long)p.AS * 2 * p.a_slot) / (long)raw;
    if (rs > PIX_MAX_RS) rs = PIX_MAX_RS;
    if (rs < 3) return fail(TAGI_ERR_UNSUPPORTED, "patch too large for the shared-memory rings");
    p.RS = (int)rs;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (unsigned)plan.col_tiles, (unsigned)plan.row_pairs, 1);
    cfg.blockDim = dim3(32 * (3 + NCW));
    cfg.stream = st;
    cfg.dynamicSmemBytes = pix_smem<OP>(p.a_slot, p.AS, p.RS, DS);
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    cudaError_t e;
#define TAGI_PIX_LAUNCH(CHV, RELUV)                                                                              \
    do {                                                                                                         \
        auto kfn = tagi_tc_conv_pix_kernel<OP, CHV, DS, ACC, RELUV, NCW>;                                             \
        e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);                  \
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute");                                       \
        e = cudaLaunchKernelEx(&cfg, kfn, a0, a1, b0, b1, p, plan.bn, status);                                   \
    } while (0)
    if (OP == OP_FWD && relu) {
        if (tc_chunked()) TAGI_PIX_LAUNCH(CHUNK_STAGES, true); else TAGI_PIX_LAUNCH(0, true);
    } else {
        if (tc_chunked()) TAGI_PIX_LAUNCH(CHUNK_STAGES, false); else TAGI_PIX_LAUNCH(0, false);
    }
#undef TAGI_PIX_LAUNCH
    if (e != cudaSuccess) return cuda_fail(e, "implicit Conv2d kernel launch");
    return TAGI_OK;
}

}  // namespace

bool conv_param_patch_supported(const tagi_conv2d_geom &g, std::initializer_list<const void *> ptrs) {
    for (const void *q : ptrs)
        if (q && !aligned16(q)) return false;
    ParamPlan plan;
    return plan_param(g, &plan);
}

size_t conv_param_patch_workspace_bytes(const tagi_conv2d_geom &g) {
    ParamPlan plan;
    if (!plan_param(g, &plan)) return 0;
    return plan.slices > 1 ? (size_t)2 * plan.slices * g.fo * plan.pp.Kc * sizeof(float) : 0;
}

int conv2d_bwd_param_patch(const tagi_conv2d_geom &g, const float *var_w, const float *mu_a, const float *dmu_z,
                           const float *dvar_z, float *dmu_w, float *dvar_w, cudaStream_t st) {
    ParamPlan plan;
    if (!plan_param(g, &plan)) return fail(TAGI_ERR_UNSUPPORTED, "Conv2d geometry not supported by the implicit parameter pass");
    PatchParam &p = plan.pp;
    int *status = tc_status_word();
    if (!status) return fail(TAGI_ERR_CUDA, "cannot allocate the tensor-core status word");
    CUtensorMap tx, td0, td1;
    int rc;
    // flat mode: the plane is one row of H * W pixels
    const int mw = p.flat ? g.hi * g.wi : g.wi, mh = p.flat ? 1 : g.hi, ow = p.flat ? g.ho * g.wo : g.wo, oh = p.flat ? 1 : g.ho;
    if ((rc = make_tmap_nchw(&tx, mu_a, mw, mh, g.fi, g.B, p.PW, p.flat ? 1 : g.k, p.CT, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
    // a CTA stages exactly the output channels it needs: half of the pair's, or all of a single CTA's
    const unsigned brows = plan.pair ? plan.bn / 2 : plan.bn;
    const CUtensorMapSwizzle bswz = plan.sk == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
    if ((rc = make_tmap_nchw(&td0, dmu_z, ow, oh, g.fo, g.B, plan.sk, 1, brows, bswz))) return rc;
    if ((rc = make_tmap_nchw(&td1, dvar_z, ow, oh, g.fo, g.B, plan.sk, 1, brows, bswz))) return rc;
    const long slice = (long)g.fo * p.Kc;
    p.slice_elems = slice;
    if (plan.slices > 1) {
        float *ws = nullptr;
        if ((rc = conv_scratch((size_t)2 * plan.slices * slice * sizeof(float), &ws, st)) != TAGI_OK) return rc;
        p.out1 = ws, p.out2 = ws + (long)plan.slices * slice, p.scale = nullptr;
    } else {
        p.out1 = dmu_w, p.out2 = dvar_w, p.scale = var_w;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = plan.pair ? dim3(2 * (unsigned)plan.col_tiles, (unsigned)plan.row_pairs, (unsigned)plan.slices)
                            : dim3((unsigned)plan.col_tiles, (unsigned)plan.row_tiles, (unsigned)plan.slices);
    cfg.blockDim = dim3(NTHREADS2 - 32);
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = plan.pair ? 2 : 1;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaSuccess;
    // ring depths: RS raw slots (patch + two delta tiles), DS slots of A operands in tensor memory, which holds the two
    // accumulators (ACC columns each) and DS * 64 columns of A operands: six slots when the output tile is at most 64 wide
    // (measured: deeper rings change nothing; the pass is bound by the converter warps' instruction stream)
#define TAGI_PATCH_LAUNCH(CHV, RSV, DSV, ACCV, NCWV, PAIRV, KSV)                                                 \
    do {                                                                                                         \
        auto kfn = tagi_tc_conv_param_kernel<CHV, RSV, DSV, ACCV, NCWV, PAIRV, KSV>;                             \
        cfg.blockDim = dim3(32 * (3 + NCWV));                                                                    \
        cfg.dynamicSmemBytes = patch_param_smem<RSV, DSV, KSV>(p.a_slot);                                        \
        if (cfg.dynamicSmemBytes > 227 * 1024) return fail(TAGI_ERR_UNSUPPORTED, "patch too large for the shared-memory ring"); \
        e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);                  \
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute");                                       \
        e = cudaLaunchKernelEx(&cfg, kfn, tx, td0, td1, p, plan.bn, status);                                     \
    } while (0)
    // chunk of the accumulation: 256 contraction steps = 16 slabs of 16 pixels or 8 slabs of 32
    const bool ch = tc_chunked() != 0;
    if (plan.sk == 32) {
        if (plan.bn <= 64 && !plan.pair) { if (ch) TAGI_PATCH_LAUNCH(8, 5, 3, 64, 8, false, 4); else TAGI_PATCH_LAUNCH(0, 5, 3, 64, 8, false, 4); }
        else if (plan.bn <= 64) { if (ch) TAGI_PATCH_LAUNCH(8, 5, 3, 64, 8, true, 4); else TAGI_PATCH_LAUNCH(0, 5, 3, 64, 8, true, 4); }
        else { if (ch) TAGI_PATCH_LAUNCH(8, 5, 2, 128, 8, true, 4); else TAGI_PATCH_LAUNCH(0, 5, 2, 128, 8, true, 4); }
    } else {
        if (plan.bn <= 64 && !plan.pair) { if (ch) TAGI_PATCH_LAUNCH(16, 6, 6, 64, 8, false, 2); else TAGI_PATCH_LAUNCH(0, 6, 6, 64, 8, false, 2); }
        else if (plan.bn <= 64) { if (ch) TAGI_PATCH_LAUNCH(16, 6, 6, 64, 8, true, 2); else TAGI_PATCH_LAUNCH(0, 6, 6, 64, 8, true, 2); }
        else { if (ch) TAGI_PATCH_LAUNCH(16, 6, 4, 128, 8, true, 2); else TAGI_PATCH_LAUNCH(0, 6, 4, 128, 8, true, 2); }
    }
#undef TAGI_PATCH_LAUNCH
    if (e != cudaSuccess) return cuda_fail(e, "implicit Conv2d parameter pass launch");
    if (plan.slices > 1) {
        patch_reduce_slices_kernel<<<(unsigned)((slice + 255) / 256), 256, 0, st>>>(p.out1, p.out2, var_w, slice, plan.slices,
                                                                                    dmu_w, dvar_w);
        e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_fail(e, "patch_reduce_slices_kernel launch");
    }
    return TAGI_OK;
}

bool conv_pix_patch_supported(const tagi_conv2d_geom &g, int pass, std::initializer_list<const void *> ptrs) {
    for (const void *q : ptrs)
        if (q && !aligned16(q)) return false;
    PixPlan plan;
    return plan_pix(g, pass, &plan);
}

size_t conv_pix_patch_workspace_bytes(const tagi_conv2d_geom &g) {
    return (size_t)2 * g.fo * g.fi * g.k * g.k * sizeof(float);   // the regrouped weights (means and variances)
}

int conv2d_fwd_patch(const tagi_conv2d_geom &g, const float *mu_w, const float *var_w, const float *mu_b, const float *var_b,
                     const float *mu_a, const float *var_a, float *mu_z, float *var_z, cudaStream_t st, float *relu_jcb) {
    PixPlan plan;
    if (!plan_pix(g, CONV_PASS_FWD, &plan)) return fail(TAGI_ERR_UNSUPPORTED, "Conv2d geometry not supported by the implicit forward pass");
    PixParam &p = plan.pp;
    const long nw = (long)g.fo * g.fi * p.k2;
    float *ws = nullptr;
    int rc = conv_scratch((size_t)2 * nw * sizeof(float), &ws, st);
    if (rc != TAGI_OK) return rc;
    const long blocks = (nw + 255) / 256;
    regroup_weights_fwd_kernel<<<(unsigned)(blocks < 148 * 8 ? blocks : 148 * 8), 256, 0, st>>>(mu_w, var_w, g.fo, g.fi, p.k2, ws,
                                                                                             ws + nw);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "regroup_weights_fwd_kernel launch");
    CUtensorMap a0, a1, b0, b1;
    if ((rc = make_tmap_nchw(&a0, mu_a, g.wi, g.hi, g.fi, g.B, p.PW, p.PR, 16, CU_TENSOR_MAP_SWIZZLE_NONE, p.NI))) return rc;
    if ((rc = make_tmap_nchw(&a1, var_a, g.wi, g.hi, g.fi, g.B, p.PW, p.PR, 16, CU_TENSOR_MAP_SWIZZLE_NONE, p.NI))) return rc;
    if ((rc = make_tmap_weights(&b0, ws, (uint64_t)g.fi * p.k2, g.fo, false, plan.bn / 2))) return rc;
    if ((rc = make_tmap_weights(&b1, ws + nw, (uint64_t)g.fi * p.k2, g.fo, false, plan.bn / 2))) return rc;
    p.out1 = mu_z, p.out2 = var_z, p.out3 = relu_jcb, p.aux1 = mu_b, p.aux2 = var_b;
    // (sixteen converter warps were measured on the 64-column tiles: no gain in the forward pass, 8 % in the state pass)
    if (plan.bn <= 64) return launch_pix<OP_FWD, 4, 64, 8>(a0, a1, b0, b1, plan, relu_jcb != nullptr, st);
    if (plan.bn <= 112) return launch_pix<OP_FWD, 3, 112, 8>(a0, a1, b0, b1, plan, relu_jcb != nullptr, st);
    return launch_pix<OP_FWD, 2, 128, 8>(a0, a1, b0, b1, plan, relu_jcb != nullptr, st);
}

int conv2d_bwd_state_patch(const tagi_conv2d_geom &g, const float *mu_w, const float *jcb, const float *dmu_z,
                           const float *dvar_z, float *dmu_a, float *dvar_a, cudaStream_t st) {
    PixPlan plan;
    if (!plan_pix(g, CONV_PASS_STATE, &plan)) return fail(TAGI_ERR_UNSUPPORTED, "Conv2d geometry not supported by the implicit state pass");
    PixParam &p = plan.pp;
    const long nw = (long)g.fo * g.fi * p.k2;
    float *ws = nullptr;
    int rc = conv_scratch((size_t)nw * sizeof(float), &ws, st);
    if (rc != TAGI_OK) return rc;
    const long blocks = (nw + 255) / 256;
    regroup_weights_state_kernel<<<(unsigned)(blocks < 148 * 8 ? blocks : 148 * 8), 256, 0, st>>>(mu_w, g.fo, g.fi, p.k2, ws);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "regroup_weights_state_kernel launch");
    CUtensorMap a0, a1, b0;
    if ((rc = make_tmap_nchw(&a0, dmu_z, g.wo, g.ho, g.fo, g.B, p.PW, p.PR, 16, CU_TENSOR_MAP_SWIZZLE_NONE, p.NI))) return rc;
    if ((rc = make_tmap_nchw(&a1, dvar_z, g.wo, g.ho, g.fo, g.B, p.PW, p.PR, 16, CU_TENSOR_MAP_SWIZZLE_NONE, p.NI))) return rc;
    if ((rc = make_tmap_weights(&b0, ws, g.fi, (uint64_t)g.fo * p.k2, true))) return rc;
    p.out1 = dmu_a, p.out2 = dvar_a, p.out3 = nullptr, p.aux1 = jcb, p.aux2 = nullptr;
    if (plan.bn <= 64) return launch_pix<OP_BWD_STATE, 6, 64, 16>(a0, a1, b0, b0, plan, false, st);
    // wider tiles: sixteen converter warps as well, each with a 32-column slice of the accumulators (measured on ResNet-18
    // layer2, 128 columns: 0.309 ms with eight warps, 0.272 ms with sixteen)
    return launch_pix<OP_BWD_STATE, 4, 128, 16>(a0, a1, b0, b0, plan, false, st);
}

}  // namespace tagi
