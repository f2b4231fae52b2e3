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
#include "tagi_tc_tile.cuh"

namespace tagi {
namespace {

struct PatchParam {
    int fi, k, k2, Kc, fo;
    int CT;               // channels per CTA row tile
    int ho, nxc;          // output rows per image, 16-pixel chunks per output row
    int stride, PW, lead; // patch row pitch in floats; a row's first useful column
    int x0, y0;           // patch origin relative to (ox0 * stride, oy * stride): -(off + lead), -off
    int total_slabs, slabs_per_slice;
    uint32_t a_bytes;     // bytes of the patch box
    uint32_t a_slot;      // ring slot reserved for it (multiple of 1024)
    float *out1, *out2;   // [slice][fo][Kc]
    const float *scale;   // var_w when the contraction is not sliced, else null (raw partial sums)
    long slice_elems;
};

constexpr int P_NA = 4, P_NRAW_B = 2, P_NDER = 2;

template <int RS, int DS>
size_t patch_param_smem(uint32_t a_slot) {
    return (size_t)RS * (a_slot + P_NRAW_B * HALF_BYTES) + (size_t)DS * P_NDER * HALF_BYTES + 1024 + 256;
}

template <int CH, int RS, int DS>
__global__ void __launch_bounds__(NTHREADS2 - 32, 1)
tagi_tc_conv_param_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmD0,
                          const __grid_constant__ CUtensorMap tmD1, const PatchParam pp, const int bn, int *status) {
    constexpr int NA = P_NA, NDER = P_NDER;
    constexpr uint32_t DER_SLOT = NDER * HALF_BYTES;
    constexpr uint32_t NCOLS = 512;
    constexpr uint32_t acc_stride = 128, A_COL0 = 256;
    static_assert(A_COL0 + DS * NA * BK <= 512, "tensor memory: accumulators + A slots");
    const uint32_t RAW_SLOT = pp.a_slot + P_NRAW_B * HALF_BYTES;
    const uint32_t IDESC = make_idesc_tf32(256, bn, 0, 0);

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
    const uint32_t cta = cluster_ctarank();  // 0 issues the MMAs
    const int half = bn / 2;
    const int tile = blockIdx.y * 2 + (int)cta;                   // this CTA's row tile: channels c0 .. c0 + CT - 1
    const int c0 = tile * pp.CT;
    const int col0 = (blockIdx.x >> 1) * bn;                      // the pair's output channels
    const int brow0 = col0 + (int)cta * half;                     // this CTA's half of them (B rows)
    const int kb = (int)blockIdx.z * pp.slabs_per_slice;          // first slab of this slice
    const int nk = min(pp.total_slabs - kb, pp.slabs_per_slice);
    const int chunk_len = CH > 0 ? CH : nk;

    if (threadIdx.x == 0) {
        for (int s = 0; s < RS; s++) mbar_init(raw_full + s, 1);
        for (int s = 0; s < L; s++) mbar_init(stage_done + s, 2);            // one commit from each MMA issuer
        for (int s = 0; s < DS; s++) mbar_init(conv_done + s, NCONV_WARPS);  // used in CTA 0: one warp group of each CTA
        mbar_init(acc_full, 2);
        mbar_init(acc_empty, 2 * NCONV_WARPS);                              // used in CTA 0 only
        *abort_flag = 0;
        mbar_init_fence();
        prefetch_tmap(&tmX);
        prefetch_tmap(&tmD0);
        prefetch_tmap(&tmD1);
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot, NCOLS);
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers exist before anyone arrives on them
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
                const int t = kb + it;                                  // slab -> (image, output row, 16-pixel chunk)
                const int xc = t % pp.nxc, rr = t / pp.nxc, oy = rr % pp.ho, b = rr / pp.ho;
                mbar_arrive_expect_tx(raw_full + r, pp.a_bytes + P_NRAW_B * HALF_BYTES);
                const uint32_t st = raw_base + r * RAW_SLOT;
                tma_load_4d(st, &tmX, xc * 16 * pp.stride + pp.x0, oy * pp.stride + pp.y0, c0, b, raw_full + r);
                tma_load_4d(st + pp.a_slot, &tmD0, xc * 16, oy, brow0, b, raw_full + r);
                tma_load_4d(st + pp.a_slot + HALF_BYTES, &tmD1, xc * 16, oy, brow0, b, raw_full + r);
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
                const uint32_t rb = raw_base + r * RAW_SLOT + pp.a_slot, ds = der_base + d * DER_SLOT;
                const uint32_t at = tmem + A_COL0 + d * (NA * BK);
                constexpr uint32_t LBO = 16, KSTEP = 32 >> 4;
                constexpr uint32_t HI = desc_hi(512, SWZ_64B);
                const uint32_t rbl = desc_lo(rb, LBO), dsl = desc_lo(ds, LBO);
                if (chain1) {
                    mma_kstep_cparam_pair<1>(d1, d2, at, rbl, dsl, HI, IDESC, f, f);
                    mma_kstep_cparam_pair<1>(d1, d2, at + 8, rbl + KSTEP, dsl + KSTEP, HI, IDESC, 1, 1);
                } else {
                    mma_kstep_cparam_pair<2>(d1, d2, at, rbl, dsl, HI, IDESC, f, f);
                    mma_kstep_cparam_pair<2>(d1, d2, at + 8, rbl + KSTEP, dsl + KSTEP, HI, IDESC, 1, 1);
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
        // this thread's row (channel cl of the tile, tap ky, kx): byte offset of its first value inside the patch.
        // Rows past the tile's CT * k * k read the patch's first values: finite numbers whose sums are never stored.
        const bool row_in_tile = arow < pp.CT * pp.k2;
        uint32_t row_off = 0;
        {
            const int m = row_in_tile ? arow : 0;
            const int cl = m / pp.k2, tap = m - cl * pp.k2, ky = tap / pp.k, kx = tap - ky * pp.k;
            row_off = (uint32_t)(((cl * pp.k + ky) * pp.PW + kx + pp.lead) * 4);
        }
        const uint32_t step_b = (uint32_t)pp.stride * 4;
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
            if (lane == 0) mbar_arrive_cluster(acc_empty, 0);
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
        for (int it = h; it < nk && ok; it += 2) {
            const int r = it % RS, d = it % DS;
            ok = mbar_wait(raw_full + r, (it / RS) & 1, abort_flag, status, ST_TIMEOUT_RAW) &&
                 (it < DS || mbar_wait(stage_done + (it - DS) % L, ((it - DS) / L) & 1, abort_flag, status,
                                       ST_TIMEOUT_EMPTY));
            if (!ok) break;
            const uint32_t rs = raw_base + r * RAW_SLOT, rb = rs + pp.a_slot, ds = der_base + d * DER_SLOT;

#pragma unroll
            for (int kh = 0; kh < 2; kh++) {  // the two 8-wide k steps: pixels kh*8 .. kh*8+7 of the slab
                float x[8];
#pragma unroll
                for (int i = 0; i < 8; i++)
                    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(x[i]) : "r"(rs + row_off + (kh * 8 + i) * step_b));
                const uint32_t at = lane_addr + A_COL0 + d * (NA * BK) + kh * 8;
                float t0[8], t1[8], qq[8];
#pragma unroll
                for (int i = 0; i < 8; i++) qq[i] = x[i] * x[i], t0[i] = hi_part(x[i]), t1[i] = hi_part(qq[i]);
                tmem_st_32x8(at + 0 * BK, t0);
                tmem_st_32x8(at + 1 * BK, t1);
#pragma unroll
                for (int i = 0; i < 8; i++) t0[i] = x[i] - t0[i], t1[i] = qq[i] - t1[i];
                tmem_st_32x8(at + 2 * BK, t0);
                tmem_st_32x8(at + 3 * BK, t1);
            }
            // B halves (dmu_z, dvar_z tiles of this CTA's 64 channels): lo parts at the same swizzled offsets
#pragma unroll
            for (int c = 0; c < 2; c++) {
                const uint32_t o = gt * 16 + c * (HALF_BYTES / 2);
                const float4 b0 = lds128(rb + o), b1 = lds128(rb + HALF_BYTES + o);
                sts128(ds + 0 * HALF_BYTES + o, lo_part(b0));
                sts128(ds + 1 * HALF_BYTES + o, lo_part(b1));
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

        // epilogue: row (c, tap) of the tile is weight column kc = c0 * k2 + arow; this thread holds 64 output channels
        // of it. out[co][kc]: for one co the 32 lanes of a warp write 32 consecutive kc (coalesced).
        const int kc = c0 * pp.k2 + arow;
        if (ok && row_in_tile && kc < pp.Kc) {
            float *o1 = pp.out1 + (long)blockIdx.z * pp.slice_elems + kc;
            float *o2 = pp.out2 + (long)blockIdx.z * pp.slice_elems + kc;
            const int cbase = col0 + h * 64, valid = min(bn - h * 64, pp.fo - cbase);
#pragma unroll
            for (int i0 = 0; i0 < 64; i0 += 8) {
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

// 4-D tensor map over a [B][C][H][W] FP32 tensor
int make_tmap_nchw(CUtensorMap *tm, const float *ptr, int W, int H, int C, int B, unsigned bx, unsigned by, unsigned bc,
                   CUtensorMapSwizzle swz) {
    EncodeTiledFn fn = tc_encode_fn();
    if (!fn) return fail(TAGI_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[4] = {(cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)C, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)W * 4, (cuuint64_t)W * H * 4, (cuuint64_t)W * H * C * 4};
    cuuint32_t box[4] = {bx, by, bc, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(TAGI_ERR_CUDA, "cuTensorMapEncodeTiled (4-D) failed with code " + std::to_string((int)r));
    return TAGI_OK;
}

struct ParamPlan {
    PatchParam pp;
    int bn, col_tiles, row_pairs, slices;
};

inline int round_up4(int v) { return (v + 3) & ~3; }

bool plan_param(const tagi_conv2d_geom &g, ParamPlan *out) {
    const int off = g.pad_type == 1 ? g.pad : 0;
    const int k2 = g.k * g.k;
    if (k2 > 128 || g.wi % 4 || g.wo % 4 || g.fo < 16) return false;
    PatchParam &p = out->pp;
    p.fi = g.fi, p.k = g.k, p.k2 = k2, p.Kc = k2 * g.fi, p.fo = g.fo;
    p.CT = 128 / k2 < g.fi ? 128 / k2 : g.fi;
    p.ho = g.ho, p.nxc = (g.wo + 15) / 16;
    p.stride = g.stride;
    p.lead = round_up4(off) - off;
    p.x0 = -round_up4(off), p.y0 = -off;
    p.PW = round_up4(15 * g.stride + g.k + p.lead);
    if (p.PW > 256 || p.CT > 256 || g.k > 256) return false;
    p.a_bytes = (uint32_t)p.PW * g.k * p.CT * 4;
    p.a_slot = (p.a_bytes + 1023u) & ~1023u;
    if (p.a_slot > 24 * 1024) return false;
    const long total = (long)g.B * g.ho * p.nxc;
    if (total >= (1L << 31)) return false;
    p.total_slabs = (int)total;
    // output channels per pair: one tile when it fits, else the width that wastes least
    int bn = g.fo <= 128 ? ((g.fo + 15) / 16) * 16 : 128;
    if (g.fo > 128) {
        long best = -1;
        for (int w = 128; w >= 64; w -= 16) {
            const long waste = (long)((g.fo + w - 1) / w) * w - g.fo;
            if (best < 0 || waste < best) best = waste, bn = w;
        }
    }
    out->bn = bn;
    out->col_tiles = (g.fo + bn - 1) / bn;
    const int row_tiles = (g.fi + p.CT - 1) / p.CT;
    out->row_pairs = (row_tiles + 1) / 2;
    // slices: about one wave of CTA pairs (two when the contraction is long), at least 32 slabs each
    const long pairs = (long)out->row_pairs * out->col_tiles;
    const int slots = tc_sm_budget() / 2;
    long s = pairs >= slots ? 1 : slots / pairs;
    if (s > total / 32) s = total / 32;
    if (s < 1) s = 1;
    p.slabs_per_slice = (int)((total + s - 1) / s);
    out->slices = (int)((total + p.slabs_per_slice - 1) / p.slabs_per_slice);
    return true;
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
    if ((rc = make_tmap_nchw(&tx, mu_a, g.wi, g.hi, g.fi, g.B, p.PW, g.k, p.CT, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
    if ((rc = make_tmap_nchw(&td0, dmu_z, g.wo, g.ho, g.fo, g.B, 16, 1, 64, CU_TENSOR_MAP_SWIZZLE_64B))) return rc;
    if ((rc = make_tmap_nchw(&td1, dvar_z, g.wo, g.ho, g.fo, g.B, 16, 1, 64, CU_TENSOR_MAP_SWIZZLE_64B))) return rc;
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
    cfg.gridDim = dim3(2 * (unsigned)plan.col_tiles, (unsigned)plan.row_pairs, (unsigned)plan.slices);
    cfg.blockDim = dim3(NTHREADS2 - 32);
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    constexpr int RS = 6, DS = 4;
    cfg.dynamicSmemBytes = patch_param_smem<RS, DS>(p.a_slot);
    if (cfg.dynamicSmemBytes > 227 * 1024) return fail(TAGI_ERR_UNSUPPORTED, "patch too large for the shared-memory ring");
    cudaError_t e;
#define TAGI_PATCH_LAUNCH(CHV)                                                                                   \
    do {                                                                                                         \
        auto kfn = tagi_tc_conv_param_kernel<CHV, RS, DS>;                                                       \
        e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);                  \
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute");                                       \
        e = cudaLaunchKernelEx(&cfg, kfn, tx, td0, td1, p, plan.bn, status);                                     \
    } while (0)
    if (tc_chunked()) TAGI_PATCH_LAUNCH(CHUNK_STAGES); else TAGI_PATCH_LAUNCH(0);
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

}  // namespace tagi
