// Pieces shared by the tcgen05 kernels (tagi_linear_tc.cu, tagi_conv_patch.cu): tile constants, the epilogue
// description and the routines that turn a thread's 64 accumulated columns into stores.
#pragma once
#include <cuda.h>

#include "tagi_common.h"
#include "tagi_tc_ptx.cuh"

namespace tagi {

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time dependency on libcuda); null when the
// driver does not offer it. tc_status_word: the per-device word the kernels record a timed-out wait in.
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn tc_encode_fn();
int *tc_status_word();
int tc_sm_budget();   // SMs the tile planning counts on (tagi_tc_set_sm_budget)
int tc_chunked();     // 1: contraction accumulated in chunks of 256 (default)

namespace {

using namespace ptx;

constexpr int TM = 128, TN = 128, BK = 16;
constexpr int TILE_BYTES = 128 * BK * 4;  // 8 KiB per operand tile
constexpr int NCONV_WARPS = 8;
// epilogue staging of the ts / pair kernels: per warp two 32 x 64 blocks with a row pitch of 68 floats
constexpr uint32_t STAGE_PITCH = 68 * 4, STAGE_VALUE = 32 * STAGE_PITCH, STAGE_WARP = 2 * STAGE_VALUE;
constexpr size_t STAGE_BYTES = (size_t)NCONV_WARPS * STAGE_WARP;
__host__ __device__ constexpr size_t at_least_stage(size_t ring) { return ring > STAGE_BYTES ? ring : STAGE_BYTES; }
constexpr int NTHREADS2 = 32 * (4 + NCONV_WARPS);      // ts / pair kernels: TMA, two MMA issuers (warps 1, 10), converters,
                                                       // and warp 11, which gathers Conv2d operands (pair kernel only)
constexpr int GATHER_WARP = 3 + NCONV_WARPS;
constexpr int ISSUER2_WARP = 2 + NCONV_WARPS;
constexpr int CHUNKS = TILE_BYTES / 16;  // 16-byte chunks per tile

enum { OP_FWD = 0, OP_BWD_STATE = 1, OP_BWD_PARAM = 2 };

template <int OP> struct OpTraits;
// which operands of a pass are staged MN-major
template <> struct OpTraits<OP_FWD> { static constexpr int A_MN = 0, B_MN = 0; };
template <> struct OpTraits<OP_BWD_STATE> { static constexpr int A_MN = 0, B_MN = 1; };
template <> struct OpTraits<OP_BWD_PARAM> { static constexpr int A_MN = 1, B_MN = 1; };

struct TcEpilogue {
    float *out1, *out2;
    const float *aux1, *aux2;  // forward: bias vectors (may be null); backward: aux1 = scale matrix
    long ld;
    int rows, cols;
    // 0: outputs are row-major [rows][ld]. > 0: rows are (image, pixel) pairs with npix pixels per image, columns are
    // channels, and outputs (and the scale matrix) are laid out [image][channel][pixel] as Conv2d wants them
    int npix;
    // Split contraction: slice z = blockIdx.z covers k-slabs [z * slabs_per_slice, ...) and writes its sums at
    // out + z * slice_elems (0 slabs_per_slice: the whole contraction in one slice)
    int slabs_per_slice;
    long slice_elems;
    // Forward with the ReLU folded in (kernels instantiated with RELU only): out1 / out2 receive the moments after the
    // ReLU and out3 its Jacobian (src/activation.cpp:7-29); the pre-activation moments are not written.
    float *out3;
    // Parameter pass with the bias deltas folded in (kernels instantiated with BIAS only): bias1 / bias2 receive the
    // row sums of the two A operands (the deltas) times aux2[row] and its square
    float *bias1, *bias2;
};

// ReLU moments of one output: mu_a = max(mu_z, 0); where that is 0 the variance and the Jacobian are 0 too
__device__ __forceinline__ float relu_moments(float &m, float &v) {
    m = fmaxf(m, 0.f);
    const bool off = m == 0.f;
    v = off ? 0.f : v;
    return off ? 0.f : 1.f;
}


__device__ __forceinline__ float lo_part(float x) { return x - __uint_as_float(__float_as_uint(x) & 0xffffe000u); }
__device__ __forceinline__ float4 lo_part(float4 v) {
    return make_float4(lo_part(v.x), lo_part(v.y), lo_part(v.z), lo_part(v.w));
}
__device__ __forceinline__ float4 lds128(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, float4 v) {
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
}

// One thread's 64 columns (starting at column c0, `valid` of them inside the tile) of output row `row`:
// forward adds the bias of the column, the backward passes scale by the matrix entry (s and s*s).
template <int OP, bool RELU = false>
__device__ __forceinline__ void store_tile(const TcEpilogue &epi, int row, int c0, int valid, const float (&sum1)[64],
                                           const float (&sum2)[64]) {
    if (row >= epi.rows) return;
    if (epi.npix > 0) {
        // [image][channel][pixel]: consecutive lanes hold consecutive pixels, so each channel's store is coalesced
        const int img = row / epi.npix, pix = row - img * epi.npix;
        const long base = (long)img * epi.cols * epi.npix + pix;
        // eight columns at a time: their scale entries are loaded together, so that the epilogue waits for memory once
        // per group and not once per column
#pragma unroll
        for (int i0 = 0; i0 < 64; i0 += 8) {
            float sc[8];
            bool ok[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int col = c0 + i0 + u;
                ok[u] = i0 + u < valid && col < epi.cols;
                sc[u] = 1.f;
                if (OP != OP_FWD && epi.aux1 && ok[u]) sc[u] = __ldg(epi.aux1 + base + (long)col * epi.npix);
            }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                if (!ok[u]) continue;
                const int col = c0 + i0 + u;
                const long idx = base + (long)col * epi.npix;
                float o1 = sum1[i0 + u], o2 = sum2[i0 + u];
                if (OP == OP_FWD) {
                    if (epi.aux1) {
                        o1 += __ldg(epi.aux1 + col);
                        o2 += __ldg(epi.aux2 + col);
                    }
                } else {
                    o1 *= sc[u];
                    o2 = o2 * sc[u] * sc[u];
                }
                if (RELU) __stcs(epi.out3 + idx, relu_moments(o1, o2));
                __stcs(epi.out1 + idx, o1);
                __stcs(epi.out2 + idx, o2);
            }
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < 64; i += 4) {
        const int col = c0 + i;
        if (i >= valid || col >= epi.cols) break;  // tile widths and cols are multiples of 4 on this path
        const long idx = (long)row * epi.ld + col;
        float4 o1 = make_float4(sum1[i], sum1[i + 1], sum1[i + 2], sum1[i + 3]);
        float4 o2 = make_float4(sum2[i], sum2[i + 1], sum2[i + 2], sum2[i + 3]);
        if (OP == OP_FWD) {
            if (epi.aux1) {
                const float4 b1 = __ldg(reinterpret_cast<const float4 *>(epi.aux1 + col));
                const float4 b2 = __ldg(reinterpret_cast<const float4 *>(epi.aux2 + col));
                o1.x += b1.x, o1.y += b1.y, o1.z += b1.z, o1.w += b1.w;
                o2.x += b2.x, o2.y += b2.y, o2.z += b2.z, o2.w += b2.w;
            }
        } else if (epi.aux1) {  // no scale matrix: raw partial sums of a split contraction
            const float4 sc = __ldg(reinterpret_cast<const float4 *>(epi.aux1 + idx));
            o1.x *= sc.x, o1.y *= sc.y, o1.z *= sc.z, o1.w *= sc.w;
            o2.x = o2.x * sc.x * sc.x, o2.y = o2.y * sc.y * sc.y;
            o2.z = o2.z * sc.z * sc.z, o2.w = o2.w * sc.w * sc.w;
        }
        if (RELU) {
            float4 j;
            j.x = relu_moments(o1.x, o2.x), j.y = relu_moments(o1.y, o2.y);
            j.z = relu_moments(o1.z, o2.z), j.w = relu_moments(o1.w, o2.w);
            __stcs(reinterpret_cast<float4 *>(epi.out3 + idx), j);
        }
        __stcs(reinterpret_cast<float4 *>(epi.out1 + idx), o1);
        __stcs(reinterpret_cast<float4 *>(epi.out2 + idx), o2);
    }
}

// The same through shared memory, for row-major outputs: in tensor memory a lane owns a row, so direct stores put the 32
// lanes of an instruction on 32 different rows (32 half-used sectors per request). The warp writes its 32 x 64 block
// of both sums to `stage` (row pitch 68 floats: conflict-free 16-byte accesses both ways), then every instruction
// handles two rows with 16 lanes x 16 bytes each: scale loads and stores are contiguous 256-byte runs.
template <int OP, bool RELU = false>
__device__ __forceinline__ void store_tile_staged(const TcEpilogue &epi, uint32_t stage, int row_base, int lane, int c0,
                                                  int valid, const float (&sum1)[64], const float (&sum2)[64]) {
    const uint32_t mine = stage + lane * STAGE_PITCH;
#pragma unroll
    for (int i = 0; i < 64; i += 4) {
        sts128(mine + i * 4, make_float4(sum1[i], sum1[i + 1], sum1[i + 2], sum1[i + 3]));
        sts128(mine + STAGE_VALUE + i * 4, make_float4(sum2[i], sum2[i + 1], sum2[i + 2], sum2[i + 3]));
    }
    __syncwarp();
    const int cl = (lane & 15) * 4, col = c0 + cl;
    if (cl >= valid || col >= epi.cols) return;  // tile widths and cols are multiples of 4 on this path
    const int r0 = lane >> 4;
    const long idx0 = (long)(row_base + r0) * epi.ld + col;
    const uint32_t src = stage + r0 * STAGE_PITCH + cl * 4;
    // rows of this lane: row_base + r0 + 2 * it. The scale entries (or the bias) are fetched for all sixteen rows
    // before the first store, so that the epilogue pays the memory latency once and not once per row.
    float4 aux[16];
    if (OP == OP_FWD) {
        aux[0] = aux[1] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (epi.aux1) {
            aux[0] = __ldg(reinterpret_cast<const float4 *>(epi.aux1 + col));
            aux[1] = __ldg(reinterpret_cast<const float4 *>(epi.aux2 + col));
        }
    } else if (epi.aux1) {
#pragma unroll
        for (int it = 0; it < 16; it++)
            if (row_base + r0 + 2 * it < epi.rows)
                aux[it] = __ldg(reinterpret_cast<const float4 *>(epi.aux1 + idx0 + (long)(2 * it) * epi.ld));
    }
#pragma unroll
    for (int it = 0; it < 16; it++) {
        if (row_base + r0 + 2 * it < epi.rows) {
            const long idx = idx0 + (long)(2 * it) * epi.ld;
            float4 o1 = lds128(src + 2 * it * STAGE_PITCH), o2 = lds128(src + STAGE_VALUE + 2 * it * STAGE_PITCH);
            if (OP == OP_FWD) {
                o1.x += aux[0].x, o1.y += aux[0].y, o1.z += aux[0].z, o1.w += aux[0].w;
                o2.x += aux[1].x, o2.y += aux[1].y, o2.z += aux[1].z, o2.w += aux[1].w;
            } else if (epi.aux1) {  // no scale matrix: raw partial sums of a split contraction
                const float4 sc = aux[it];
                o1.x *= sc.x, o1.y *= sc.y, o1.z *= sc.z, o1.w *= sc.w;
                o2.x = o2.x * sc.x * sc.x, o2.y = o2.y * sc.y * sc.y;
                o2.z = o2.z * sc.z * sc.z, o2.w = o2.w * sc.w * sc.w;
            }
            if (RELU) {
                float4 j;
                j.x = relu_moments(o1.x, o2.x), j.y = relu_moments(o1.y, o2.y);
                j.z = relu_moments(o1.z, o2.z), j.w = relu_moments(o1.w, o2.w);
                __stcs(reinterpret_cast<float4 *>(epi.out3 + idx), j);
            }
            __stcs(reinterpret_cast<float4 *>(epi.out1 + idx), o1);
            __stcs(reinterpret_cast<float4 *>(epi.out2 + idx), o2);
        }
    }
}

__device__ __forceinline__ float hi_part(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }
constexpr int HALF_BYTES = TILE_BYTES / 2;  // B half tile: 64 rows x 16 k

// Contraction chunk: CHUNK_STAGES k-slabs (256 k) accumulate in one tensor-memory set before they are
// added to the register sums. CHUNK_STAGES == 0 (template) means a single chunk: everything stays in set 0.
constexpr int CHUNK_STAGES = 16;

template <int OP> struct PairTraits;
// raw slot: A0 A1 (8 KiB each) then B halves (4 KiB each); derived slot: B halves only
template <> struct PairTraits<OP_FWD> { static constexpr int NRAW_B = 2, NDER = 4, NA = 6; };
template <> struct PairTraits<OP_BWD_STATE> { static constexpr int NRAW_B = 1, NDER = 3, NA = 4; };
template <> struct PairTraits<OP_BWD_PARAM> { static constexpr int NRAW_B = 1, NDER = 3, NA = 4; };


// B half tile: K-major one box of 64 rows; MN-major two boxes of 32 rows
template <int MN>
__device__ __forceinline__ void load_half_tile(uint32_t dst, const CUtensorMap *tm, int row0, int k0, uint64_t *bar) {
    if (MN) {
#pragma unroll
        for (int g = 0; g < 2; g++) tma_load_2d(dst + g * 2048, tm, row0 + 32 * g, k0, bar);
    } else {
        tma_load_2d(dst, tm, k0, row0, bar);
    }
}

}  // namespace
}  // namespace tagi
