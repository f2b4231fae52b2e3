// FP32 FFMA tile engine for the TAGI contractions (sm_100a).
//
// One kernel template serves Linear and Conv2d, forward and both backward passes. All of
// them have the shape
//     c1[m][n] = sum_k a1(m,k) * b1(n,k)
//     c2[m][n] = sum_k a2(m,k) * b2(n,k)  (+ a3(m,k) * b3(n,k) for the forward variance)
// where the a* / b* values are derived from the tensors in HBM while a tile is staged
// (squares, mu^2 + var), so no derived tensor is ever written to memory.
//
// A CTA owns a BM x BN output tile. Per k-slab of BK it keeps the derived operand values in
// shared memory as [array][k][row] (row-contiguous, so each thread reads its 4-row groups with
// one 16-byte load), double-buffered; the next slab is fetched from global memory into
// registers while the current one is multiplied. Each thread holds a TM x TN micro-tile of
// both accumulators in registers.
#pragma once
#include <cuda_runtime.h>

namespace tagi {

// How a thread block reads an operand tile (rows x BK) from global memory.
enum LoadMode {
    LOAD_K_VEC4 = 0,    // contraction index contiguous in memory, 16-byte loads along k
    LOAD_R_VEC4 = 1,    // row index contiguous in memory, 16-byte loads along rows
    LOAD_K_SCALAR = 2,  // 4-byte loads, lanes walk k fastest (any alignment, gathers)
    LOAD_R_SCALAR = 3   // 4-byte loads, lanes walk rows fastest
};

struct TileL {  // large problems
    static constexpr int BM = 128, BN = 128, BK = 8, TM = 8, TN = 8, NT = 256;
};
struct TileS {  // small or skinny problems
    static constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4, NT = 256;
};

// ---------------------------------------------------------------------------------------
// Derivation of the staged values from the raw tensors
// ---------------------------------------------------------------------------------------
enum Derive {
    DER_MEAN_VAR_ACT = 0,  // (x0, x1) -> (x0, x0*x0 + x1, x1)   forward activations: mu_a, mu_a^2+var_a, var_a
    DER_MEAN_VAR_W = 1,    // (x0, x1) -> (x0, x1, x0*x0)        forward weights:     mu_w, var_w, mu_w^2
    DER_PAIR = 2,          // (x0, x1) -> (x0, x1)               deltas
    DER_SQUARE = 3         // (x0)     -> (x0, x0*x0)            mu_w / mu_a in the backward passes
};
template <int D> struct DeriveTraits;
template <> struct DeriveTraits<DER_MEAN_VAR_ACT> { static constexpr int NSRC = 2, NSM = 3; };
template <> struct DeriveTraits<DER_MEAN_VAR_W> { static constexpr int NSRC = 2, NSM = 3; };
template <> struct DeriveTraits<DER_PAIR> { static constexpr int NSRC = 2, NSM = 2; };
template <> struct DeriveTraits<DER_SQUARE> { static constexpr int NSRC = 1, NSM = 2; };

template <int D>
__device__ __forceinline__ void derive(float x0, float x1, float (&v)[DeriveTraits<D>::NSM]) {
    if (D == DER_MEAN_VAR_ACT) {
        v[0] = x0;
        v[1] = fmaf(x0, x0, x1);
        v[2] = x1;
    } else if (D == DER_MEAN_VAR_W) {
        v[0] = x0;
        v[1] = x1;
        v[2] = x0 * x0;
    } else if (D == DER_PAIR) {
        v[0] = x0;
        v[1] = x1;
    } else {
        v[0] = x0;
        v[1] = x0 * x0;
    }
}

// ---------------------------------------------------------------------------------------
// Operands
// ---------------------------------------------------------------------------------------
// Dense strided operand: element (r, k) of source s lives at src[s][r * ld_r + k * ld_k];
// exactly one of ld_r / ld_k is 1 for the vector modes.
template <int D>
struct StridedOperand {
    static constexpr int NSRC = DeriveTraits<D>::NSRC, NSM = DeriveTraits<D>::NSM;
    static constexpr int DER = D;
    const float *src0, *src1;
    long ld_r, ld_k;
    int rows, kdim;
    struct Ctx {
        long base;
        bool ok;
    };
    __device__ __forceinline__ Ctx row_ctx(int r) const { return {(long)r * ld_r, r < rows}; }
    __device__ __forceinline__ void load(const Ctx &c, int k, float (&v)[NSM]) const {
        float x0 = 0.f, x1 = 0.f;
        if (c.ok && k < kdim) {
            long i = c.base + (long)k * ld_k;
            x0 = __ldg(src0 + i);
            if (NSRC == 2) x1 = __ldg(src1 + i);
        }
        derive<D>(x0, x1, v);
    }
    // four consecutive elements along the contiguous index starting at (r, k)
    __device__ __forceinline__ void load4(int r, int k, float4 &x0, float4 &x1) const {
        x0 = make_float4(0.f, 0.f, 0.f, 0.f);
        x1 = x0;
        if (r < rows && k < kdim) {
            long i = (long)r * ld_r + (long)k * ld_k;
            x0 = __ldg(reinterpret_cast<const float4 *>(src0 + i));
            if (NSRC == 2) x1 = __ldg(reinterpret_cast<const float4 *>(src1 + i));
        }
    }
};

// ---------------------------------------------------------------------------------------
// Tile staging: global -> registers -> (derive) -> shared
// ---------------------------------------------------------------------------------------
template <class Cfg, int ROWS, class Op, int MODE>
struct Stager {
    static constexpr int BK = Cfg::BK, NT = Cfg::NT, LD = ROWS + 4;
    static constexpr int NSM = Op::NSM;
    static constexpr int EPT = ROWS * BK / NT;  // elements per thread per smem array
    static_assert(EPT == 4, "tile shape must give 4 elements per thread");
    static constexpr int NCTX = (MODE == LOAD_K_SCALAR) ? EPT : 1;

    float regs[NSM][EPT];
    typename Op::Ctx ctx[NCTX];

    __device__ __forceinline__ void init(const Op &op, int row0) {
        const int tid = threadIdx.x;
        if constexpr (MODE == LOAD_K_SCALAR) {
#pragma unroll
            for (int i = 0; i < EPT; i++) ctx[i] = op.row_ctx(row0 + tid / BK + i * (NT / BK));
        } else if constexpr (MODE == LOAD_R_SCALAR) {
            ctx[0] = op.row_ctx(row0 + tid % ROWS);
        }
    }

    __device__ __forceinline__ void fetch(const Op &op, int row0, int k0) {
        const int tid = threadIdx.x;
        if constexpr (MODE == LOAD_K_VEC4) {
            constexpr int CPR = BK / 4;  // 16-byte chunks per row
            float4 x0, x1;
            op.load4(row0 + tid / CPR, k0 + (tid % CPR) * 4, x0, x1);
            const float a0[4] = {x0.x, x0.y, x0.z, x0.w}, a1[4] = {x1.x, x1.y, x1.z, x1.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float v[NSM];
                derive<Op::DER>(a0[i], a1[i], v);
#pragma unroll
                for (int s = 0; s < NSM; s++) regs[s][i] = v[s];
            }
        } else if constexpr (MODE == LOAD_R_VEC4) {
            constexpr int CPK = ROWS / 4;  // 16-byte chunks per k row
            float4 x0, x1;
            op.load4(row0 + (tid % CPK) * 4, k0 + tid / CPK, x0, x1);
            const float a0[4] = {x0.x, x0.y, x0.z, x0.w}, a1[4] = {x1.x, x1.y, x1.z, x1.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float v[NSM];
                derive<Op::DER>(a0[i], a1[i], v);
#pragma unroll
                for (int s = 0; s < NSM; s++) regs[s][i] = v[s];
            }
        } else if constexpr (MODE == LOAD_K_SCALAR) {
#pragma unroll
            for (int i = 0; i < EPT; i++) {
                float v[NSM];
                op.load(ctx[i], k0 + tid % BK, v);
#pragma unroll
                for (int s = 0; s < NSM; s++) regs[s][i] = v[s];
            }
        } else {
#pragma unroll
            for (int i = 0; i < EPT; i++) {
                float v[NSM];
                op.load(ctx[0], k0 + tid / ROWS + i * (NT / ROWS), v);
#pragma unroll
                for (int s = 0; s < NSM; s++) regs[s][i] = v[s];
            }
        }
    }

    // sm points at [NSM][BK][LD] for the target stage
    __device__ __forceinline__ void commit(float *sm) const {
        const int tid = threadIdx.x;
#pragma unroll
        for (int s = 0; s < NSM; s++) {
            float *base = sm + s * BK * LD;
            if constexpr (MODE == LOAD_K_VEC4) {
                constexpr int CPR = BK / 4;
                const int r = tid / CPR, kc = (tid % CPR) * 4;
#pragma unroll
                for (int i = 0; i < 4; i++) base[(kc + i) * LD + r] = regs[s][i];
            } else if constexpr (MODE == LOAD_R_VEC4) {
                constexpr int CPK = ROWS / 4;
                const int r = (tid % CPK) * 4, k = tid / CPK;
                *reinterpret_cast<float4 *>(base + k * LD + r) =
                    make_float4(regs[s][0], regs[s][1], regs[s][2], regs[s][3]);
            } else if constexpr (MODE == LOAD_K_SCALAR) {
#pragma unroll
                for (int i = 0; i < EPT; i++) base[(tid % BK) * LD + tid / BK + i * (NT / BK)] = regs[s][i];
            } else {
#pragma unroll
                for (int i = 0; i < EPT; i++) base[(tid / ROWS + i * (NT / ROWS)) * LD + tid % ROWS] = regs[s][i];
            }
        }
    }
};

template <class Cfg, int NSM>
constexpr size_t ffma_smem_bytes() {
    return (size_t)2 * NSM * Cfg::BK * ((Cfg::BM + 4) + (Cfg::BN + 4)) * sizeof(float);
}

// ---------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------
// Epi must provide:  void store(int m, int n, int z, float c1, float c2) const
//                    bool vec_ok (uniform)   and   void store4(int m, int n, int z, float4 c1, float4 c2) const
// (z = split-K slice index, 0 when the contraction is not split)
template <class Cfg, class AOp, class BOp, class Epi, int AMODE, int BMODE>
__global__ void __launch_bounds__(Cfg::NT) tagi_ffma_kernel(const AOp A, const BOp Bop, const Epi epi, const int M,
                                                            const int N, const int Kd, const int k_chunk) {
    constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, TM = Cfg::TM, TN = Cfg::TN;
    constexpr int NSM = AOp::NSM;
    static_assert(AOp::NSM == BOp::NSM, "operand arity mismatch");
    constexpr int LDA = BM + 4, LDB = BN + 4;
    constexpr int GM = TM / 4, GN = TN / 4;  // 4-wide groups per thread
    constexpr int TX = BN / TN;              // threads along n

    extern __shared__ __align__(16) float smem[];
    float *As = smem;                         // [2][NSM][BK][LDA]
    float *Bs = smem + 2 * NSM * BK * LDA;    // [2][NSM][BK][LDB]

    // n-tiles vary fastest so that concurrently running CTAs share the A rows through L2
    const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
    const int tx = threadIdx.x % TX, ty = threadIdx.x / TX;

    float c1[TM][TN], c2[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) c1[i][j] = c2[i][j] = 0.f;

    Stager<Cfg, BM, AOp, AMODE> sa;
    Stager<Cfg, BN, BOp, BMODE> sb;
    sa.init(A, m0);
    sb.init(Bop, n0);

    // split-K: slice blockIdx.z of the contraction (k_chunk is a multiple of BK; one slice when gridDim.z == 1).
    // Operands zero-fill beyond Kd, and a slice never reads into the next one because its slab count is exact.
    const int z = blockIdx.z;
    const int kb = z * k_chunk;
    const int ke = min(Kd, kb + k_chunk);
    const int nk = (ke - kb + BK - 1) / BK;
    sa.fetch(A, m0, kb);
    sb.fetch(Bop, n0, kb);
    sa.commit(As);
    sb.commit(Bs);
    __syncthreads();

    for (int kt = 0; kt < nk; kt++) {
        const int cur = kt & 1;
        if (kt + 1 < nk) {
            sa.fetch(A, m0, kb + (kt + 1) * BK);
            sb.fetch(Bop, n0, kb + (kt + 1) * BK);
        }
        const float *as = As + cur * NSM * BK * LDA;
        const float *bs = Bs + cur * NSM * BK * LDB;
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float a[NSM][TM], b[NSM][TN];
#pragma unroll
            for (int s = 0; s < NSM; s++) {
#pragma unroll
                for (int g = 0; g < GM; g++) {
                    const float4 t =
                        *reinterpret_cast<const float4 *>(as + (s * BK + kk) * LDA + g * (BM / GM) + ty * 4);
                    a[s][g * 4 + 0] = t.x, a[s][g * 4 + 1] = t.y, a[s][g * 4 + 2] = t.z, a[s][g * 4 + 3] = t.w;
                }
#pragma unroll
                for (int g = 0; g < GN; g++) {
                    const float4 t =
                        *reinterpret_cast<const float4 *>(bs + (s * BK + kk) * LDB + g * (BN / GN) + tx * 4);
                    b[s][g * 4 + 0] = t.x, b[s][g * 4 + 1] = t.y, b[s][g * 4 + 2] = t.z, b[s][g * 4 + 3] = t.w;
                }
            }
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < TN; j++) {
                    c1[i][j] = fmaf(a[0][i], b[0][j], c1[i][j]);
                    c2[i][j] = fmaf(a[1][i], b[1][j], c2[i][j]);
                    if (NSM == 3) c2[i][j] = fmaf(a[2][i], b[2][j], c2[i][j]);
                }
        }
        if (kt + 1 < nk) {
            sa.commit(As + (cur ^ 1) * NSM * BK * LDA);
            sb.commit(Bs + (cur ^ 1) * NSM * BK * LDB);
        }
        __syncthreads();
    }

    // epilogue: rows m0 + g*(BM/GM) + ty*4 + i, columns n0 + h*(BN/GN) + tx*4 + j
#pragma unroll
    for (int g = 0; g < GM; g++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int m = m0 + g * (BM / GM) + ty * 4 + i;
            if (m >= M) continue;
#pragma unroll
            for (int h = 0; h < GN; h++) {
                const int n = n0 + h * (BN / GN) + tx * 4;
                const int ri = g * 4 + i, cj = h * 4;
                if (epi.vec_ok && n + 3 < N) {
                    epi.store4(m, n, z, make_float4(c1[ri][cj], c1[ri][cj + 1], c1[ri][cj + 2], c1[ri][cj + 3]),
                               make_float4(c2[ri][cj], c2[ri][cj + 1], c2[ri][cj + 2], c2[ri][cj + 3]));
                } else {
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        if (n + j < N) epi.store(m, n + j, z, c1[ri][cj + j], c2[ri][cj + j]);
                }
            }
        }
}

// ---------------------------------------------------------------------------------------
// Epilogues for row-major outputs out[m * ld + n]
// ---------------------------------------------------------------------------------------
// out1 = c1 + bias1[n] ; out2 = c2 + bias2[n]            (Linear forward)
struct EpiRowBias {
    float *out1, *out2;
    const float *bias1, *bias2;  // may be null
    long ld;
    bool vec_ok;
    __device__ __forceinline__ void store(int m, int n, int, float c1, float c2) const {
        if (bias1) {
            c1 += __ldg(bias1 + n);
            c2 += __ldg(bias2 + n);
        }
        out1[(long)m * ld + n] = c1;
        out2[(long)m * ld + n] = c2;
    }
    __device__ __forceinline__ void store4(int m, int n, int, float4 c1, float4 c2) const {
        if (bias1) {
            const float4 b1 = __ldg(reinterpret_cast<const float4 *>(bias1 + n));
            const float4 b2 = __ldg(reinterpret_cast<const float4 *>(bias2 + n));
            c1.x += b1.x, c1.y += b1.y, c1.z += b1.z, c1.w += b1.w;
            c2.x += b2.x, c2.y += b2.y, c2.z += b2.z, c2.w += b2.w;
        }
        __stcs(reinterpret_cast<float4 *>(out1 + (long)m * ld + n), c1);
        __stcs(reinterpret_cast<float4 *>(out2 + (long)m * ld + n), c2);
    }
};

// out1 = c1 * s ; out2 = c2 * s * s, s = scale[m * ld + n]   (Jacobian in the state pass, var_w in the
// parameter pass; same association as the reference: (sum * s) * s)
struct EpiRowScale {
    float *out1, *out2;
    const float *scale;  // null: every entry is one
    long ld;
    bool vec_ok;
    __device__ __forceinline__ void store(int m, int n, int, float c1, float c2) const {
        const long i = (long)m * ld + n;
        const float s = scale ? __ldg(scale + i) : 1.f;
        out1[i] = c1 * s;
        out2[i] = c2 * s * s;
    }
    __device__ __forceinline__ void store4(int m, int n, int, float4 c1, float4 c2) const {
        const long i = (long)m * ld + n;
        const float4 s = scale ? __ldg(reinterpret_cast<const float4 *>(scale + i)) : make_float4(1.f, 1.f, 1.f, 1.f);
        c1.x *= s.x, c1.y *= s.y, c1.z *= s.z, c1.w *= s.w;
        c2.x = c2.x * s.x * s.x, c2.y = c2.y * s.y * s.y, c2.z = c2.z * s.z * s.z, c2.w = c2.w * s.w * s.w;
        __stcs(reinterpret_cast<float4 *>(out1 + i), c1);
        __stcs(reinterpret_cast<float4 *>(out2 + i), c2);
    }
};

// Split-K partial sums: slice z writes raw accumulators to part1/part2[z][m * ld + n]; a second kernel adds
// the slices in a fixed order and applies the scaling, so results do not depend on scheduling.
struct EpiPartial {
    float *part1, *part2;
    long ld, slice;  // slice = elements per slice
    bool vec_ok;
    __device__ __forceinline__ void store(int m, int n, int z, float c1, float c2) const {
        const long i = (long)z * slice + (long)m * ld + n;
        part1[i] = c1;
        part2[i] = c2;
    }
    __device__ __forceinline__ void store4(int m, int n, int z, float4 c1, float4 c2) const {
        const long i = (long)z * slice + (long)m * ld + n;
        *reinterpret_cast<float4 *>(part1 + i) = c1;
        *reinterpret_cast<float4 *>(part2 + i) = c2;
    }
};

template <class Cfg, class AOp, class BOp, class Epi, int AMODE, int BMODE>
cudaError_t launch_ffma(const AOp &A, const BOp &Bop, const Epi &epi, int M, int N, int Kd, cudaStream_t st,
                        int splits = 1) {
    auto kern = tagi_ffma_kernel<Cfg, AOp, BOp, Epi, AMODE, BMODE>;
    constexpr size_t smem = ffma_smem_bytes<Cfg, AOp::NSM>();
    if (smem > 48 * 1024) {  // opt-in is per device and per function: remember where it was done
        static bool done[64] = {};
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        if (dev < 0 || dev >= 64 || !done[dev]) {
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 64) done[dev] = true;
        }
    }
    // slice length: a multiple of BK that covers Kd in `splits` slices
    const int k_chunk = ((Kd + splits - 1) / splits + Cfg::BK - 1) / Cfg::BK * Cfg::BK;
    dim3 grid((N + Cfg::BN - 1) / Cfg::BN, (M + Cfg::BM - 1) / Cfg::BM, (Kd + k_chunk - 1) / k_chunk);
    kern<<<grid, Cfg::NT, smem, st>>>(A, Bop, epi, M, N, Kd, k_chunk);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------
// Host-side choice of tile and load modes
// ---------------------------------------------------------------------------------------
// The 128x128 tile needs enough tiles to fill the 148 SMs, otherwise the 64x64 tile gives four
// times the CTAs.
inline bool use_large_tile(int M, int N, int splits = 1) {
    if (M < 128 || N < 128) return false;
    long tiles = (long)((M + 127) / 128) * ((N + 127) / 128) * splits;
    return tiles >= 120;
}

// AM_V / AM_S: load mode of operand A when its vector path is / is not usable; same for B.
template <class AOp, class BOp, class Epi, int AM_V, int AM_S, int BM_V, int BM_S>
cudaError_t dispatch_ffma(const AOp &A, const BOp &Bo, const Epi &epi, int M, int N, int Kd, bool a_vec, bool b_vec,
                          cudaStream_t st, int splits = 1) {
    const bool big = use_large_tile(M, N, splits);
#define TAGI_GO(CFG, AM, BM_) return launch_ffma<CFG, AOp, BOp, Epi, AM, BM_>(A, Bo, epi, M, N, Kd, st, splits)
    if (big) {
        if (a_vec && b_vec) TAGI_GO(TileL, AM_V, BM_V);
        else if (a_vec) TAGI_GO(TileL, AM_V, BM_S);
        else if (b_vec) TAGI_GO(TileL, AM_S, BM_V);
        else TAGI_GO(TileL, AM_S, BM_S);
    } else {
        if (a_vec && b_vec) TAGI_GO(TileS, AM_V, BM_V);
        else if (a_vec) TAGI_GO(TileS, AM_V, BM_S);
        else if (b_vec) TAGI_GO(TileS, AM_S, BM_V);
        else TAGI_GO(TileS, AM_S, BM_S);
    }
#undef TAGI_GO
}

}  // namespace tagi
