// TAGI Conv2d on the tensor-core Linear kernels.
//
// Each pass is a gather kernel that lays the receptive fields out as a matrix in scratch memory, followed by the
// same tcgen05 3xTF32 kernel that Linear uses (tagi_linear_tc.cu), whose epilogue can write the [image][channel][pixel]
// layout directly:
//   forward         X = im2col(mu_a), im2col(var_a)  [(b, oy, ox)][ci*k*k]      -> Linear forward with the conv weights
//   state backward  stride 1: Z = gather(dmu_z), gather(dvar_z) [(b, y, x)][(co, ky, kx)] -> Linear state pass with the
//                   weights regrouped as [(co, ky, kx)][ci]
//                   stride > 1 (most entries of Z would be zeros): C = D W, D = deltas regrouped as [(b, p)][co], written
//                   as [b][(ci, ky, kx)][p], then each input pixel sums the taps that reach it and applies the Jacobian
//   parameter bwd   X = im2col(mu_a), D = deltas regrouped as [(b, p)][co]     -> Linear parameter pass
// The gathers follow the same receptive-field rule as the FFMA path (src/indices.cpp:63-104,163-194 of cuTAGI);
// taps outside the image are written as zeros. The matrices are scratch: they are consumed by the next launch on the
// same stream and never leave the device. Shapes that the tensor-core kernels cannot take (channel counts or
// fi*k*k not multiples of 4) stay on the FFMA implicit-GEMM kernels.
#include "tagi_common.h"

namespace tagi {
namespace {

struct G {
    int B, fi, hi, wi, fo, ho, wo, k, stride, off, k2, Kc, woho, wihi;
};
G geom_of(const tagi_conv2d_geom &g) {
    G q;
    q.B = g.B, q.fi = g.fi, q.hi = g.hi, q.wi = g.wi, q.fo = g.fo, q.ho = g.ho, q.wo = g.wo, q.k = g.k;
    q.stride = g.stride, q.off = g.pad_type == 1 ? g.pad : 0;
    q.k2 = g.k * g.k, q.Kc = q.k2 * g.fi, q.woho = g.wo * g.ho, q.wihi = g.wi * g.hi;
    return q;
}

// X[(b, p)][kc] = a[b][ci][oy*s - off + ky][ox*s - off + kx]; one thread per element, kc fastest (coalesced writes,
// reads of neighbouring taps hit the same cache lines). NSRC = 2 gathers mean and variance in one pass.
template <int NSRC>
__global__ void __launch_bounds__(256) im2col_kernel(const float *__restrict__ a0, const float *__restrict__ a1, G g,
                                                     float *__restrict__ x0, float *__restrict__ x1) {
    const long total = (long)g.B * g.woho * g.Kc;
    for (long t = (long)blockIdx.x * 256 + threadIdx.x; t < total; t += (long)gridDim.x * 256) {
        const int kc = (int)(t % g.Kc);
        const long n = t / g.Kc;
        const int b = (int)(n / g.woho), p = (int)(n - (long)b * g.woho);
        const int oy = p / g.wo, ox = p - oy * g.wo;
        const int ci = kc / g.k2, r = kc - ci * g.k2, ky = r / g.k, kx = r - ky * g.k;
        const int y = oy * g.stride - g.off + ky, x = ox * g.stride - g.off + kx;
        float v0 = 0.f, v1 = 0.f;
        if ((unsigned)y < (unsigned)g.hi && (unsigned)x < (unsigned)g.wi) {
            const long i = ((long)b * g.fi + ci) * g.wihi + (long)y * g.wi + x;
            v0 = __ldg(a0 + i);
            if (NSRC == 2) v1 = __ldg(a1 + i);
        }
        x0[t] = v0;
        if (NSRC == 2) x1[t] = v1;
    }
}

// Z[(b, q)][(co, ky, kx)] = delta[b][co][(y + off - ky) / s][(x + off - kx) / s] where that output pixel exists
__global__ void __launch_bounds__(256) delta_gather_kernel(const float *__restrict__ d0, const float *__restrict__ d1, G g,
                                                           float *__restrict__ z0, float *__restrict__ z1) {
    const int kd = g.fo * g.k2;
    const long total = (long)g.B * g.wihi * kd;
    for (long t = (long)blockIdx.x * 256 + threadIdx.x; t < total; t += (long)gridDim.x * 256) {
        const int kk = (int)(t % kd);
        const long n = t / kd;
        const int b = (int)(n / g.wihi), q = (int)(n - (long)b * g.wihi);
        const int y = q / g.wi, x = q - y * g.wi;
        const int co = kk / g.k2, r = kk - co * g.k2, ky = r / g.k, kx = r - ky * g.k;
        const int ty = y + g.off - ky, tx = x + g.off - kx;
        float v0 = 0.f, v1 = 0.f;
        if (ty >= 0 && tx >= 0) {
            const int oy = ty / g.stride, ox = tx / g.stride;
            if (oy * g.stride == ty && ox * g.stride == tx && oy < g.ho && ox < g.wo) {
                const long i = ((long)b * g.fo + co) * g.woho + (long)oy * g.wo + ox;
                v0 = __ldg(d0 + i);
                v1 = __ldg(d1 + i);
            }
        }
        z0[t] = v0;
        z1[t] = v1;
    }
}

// The same gathers for 2 x 2, 3 x 3 and 6 x 6 kernels, tiled through shared memory so that both sides are coalesced and no
// thread divides by a run-time number per element: a CTA stages the input patch of up to 32 output pixels
// (tx x ty of one image) for 16 channels, read along image rows, and then writes the 16 * k * k columns of each pixel
// as contiguous runs (one warp per pixel, lanes along the columns).
//   FLIP = false: X[(b, oy, ox)][(c, ky, kx)] = src[b][c][oy*s - off + ky][ox*s - off + kx]      (im2col)
//   FLIP = true : Z[(b, y, x)][(c, ky, kx)]   = src[b][c][y + off - ky][x + off - kx], stride 1  (the state pass's
//                 gather of the deltas: the same patch with the taps read in reverse)
// `g` describes the source tensor (C x H x W per image) and the pixel grid the rows run over (OH x OW).
struct TileGeom {
    int B, C, H, W, OH, OW, stride, off, tx, ty, tiles_x, tiles_y, Kc, ct;  // ct: channels staged per CTA (<= 16)
};
constexpr int GATHER_CT = 16;  // channels per CTA

constexpr int GATHER_PIX = 128;  // output pixels per CTA at most

// VEC = 4: 16-byte stores (the CTA's column count, its first column and Kc are multiples of 4); VEC = 1 otherwise.
template <int NSRC, int KS, bool FLIP, int VEC>
__global__ void __launch_bounds__(256) gather_tiled_kernel(const float *__restrict__ s0, const float *__restrict__ s1,
                                                           TileGeom g, float *__restrict__ d0, float *__restrict__ d1) {
    extern __shared__ float patch[];
    constexpr int K2 = KS * KS;
    __shared__ __align__(16) int tapoff[GATHER_CT * K2];  // column (c, ky, kx) -> offset inside the staged patch
    __shared__ int pixbase[GATHER_PIX];                    // pixel of the tile -> its window's first patch element
    __shared__ int pixrow[GATHER_PIX];                     // pixel of the tile -> row of the output matrix, -1 outside
    const int IH = (g.ty - 1) * g.stride + KS, IW = (g.tx - 1) * g.stride + KS, plane = IH * IW;
    float *p0 = patch, *p1 = patch + g.ct * plane;
    int t = blockIdx.x;
    const int tile_x = t % g.tiles_x;
    t /= g.tiles_x;
    const int tile_y = t % g.tiles_y, b = t / g.tiles_y;
    const int c0 = blockIdx.y * GATHER_CT, nc = min(GATHER_CT, g.C - c0), ncols = nc * K2, npix = g.tx * g.ty;
    const int oy0 = tile_y * g.ty, ox0 = tile_x * g.tx;
    for (int j = threadIdx.x; j < ncols; j += 256) {
        const int c = j / K2, tap = j - c * K2;
        int ky = tap / KS, kx = tap - ky * KS;
        if (FLIP) ky = KS - 1 - ky, kx = KS - 1 - kx;
        tapoff[j] = c * plane + ky * IW + kx;
    }
    for (int pix = threadIdx.x; pix < npix; pix += 256) {
        const int py = pix / g.tx, px = pix - py * g.tx, oy = oy0 + py, ox = ox0 + px;
        pixbase[pix] = (py * IW + px) * g.stride;
        pixrow[pix] = oy < g.OH && ox < g.OW ? (b * g.OH + oy) * g.OW + ox : -1;
    }
    // top-left source pixel of the patch
    const int y0 = FLIP ? oy0 + g.off - (KS - 1) : oy0 * g.stride - g.off;
    const int x0 = FLIP ? ox0 + g.off - (KS - 1) : ox0 * g.stride - g.off;
    for (int i = threadIdx.x; i < nc * plane; i += 256) {
        const int c = i / plane, r = i - c * plane, iy = r / IW, ix = r - iy * IW;
        const int y = y0 + iy, x = x0 + ix;
        float v0 = 0.f, v1 = 0.f;
        if ((unsigned)y < (unsigned)g.H && (unsigned)x < (unsigned)g.W) {
            const long a = ((long)b * g.C + c0 + c) * g.H * g.W + (long)y * g.W + x;
            v0 = __ldg(s0 + a);
            if (NSRC == 2) v1 = __ldg(s1 + a);
        }
        p0[i] = v0;
        if (NSRC == 2) p1[i] = v1;
    }
    __syncthreads();
    // one item = VEC consecutive columns of one pixel's row; items run column-fastest over the threads
    const int q = ncols / VEC;
    for (int i = threadIdx.x; i < npix * q; i += 256) {
        const int pix = i / q, jv = i - pix * q, row = pixrow[pix];
        if (row < 0) continue;
        const int pb = pixbase[pix];
        const long o = (long)row * g.Kc + (long)c0 * K2 + jv * VEC;
        if (VEC == 4) {
            const int4 a = *reinterpret_cast<const int4 *>(tapoff + 4 * jv);
            *reinterpret_cast<float4 *>(d0 + o) = make_float4(p0[pb + a.x], p0[pb + a.y], p0[pb + a.z], p0[pb + a.w]);
            if (NSRC == 2)
                *reinterpret_cast<float4 *>(d1 + o) = make_float4(p1[pb + a.x], p1[pb + a.y], p1[pb + a.z], p1[pb + a.w]);
        } else {
            const int a = tapoff[jv];
            d0[o] = p0[pb + a];
            if (NSRC == 2) d1[o] = p1[pb + a];
        }
    }
}

// W2[(co, tap)][ci] = w[co][ci][tap]: the weights with the input channel as the contiguous index
__global__ void __launch_bounds__(256) weight_regroup_kernel(const float *__restrict__ w, G g, float *__restrict__ w2) {
    const long total = (long)g.fo * g.Kc;
    for (long t = (long)blockIdx.x * 256 + threadIdx.x; t < total; t += (long)gridDim.x * 256) {
        const int ci = (int)(t % g.fi);
        const long r = t / g.fi;
        const int tap = (int)(r % g.k2), co = (int)(r / g.k2);
        w2[t] = __ldg(w + (long)co * g.Kc + ci * g.k2 + tap);
    }
}

// D[(b, p)][co] = delta[b][co][p], through a 32 x 32 shared-memory tile so that both sides are coalesced
__global__ void __launch_bounds__(256) delta_regroup_kernel(const float *__restrict__ d0, const float *__restrict__ d1, G g,
                                                            float *__restrict__ o0, float *__restrict__ o1) {
    __shared__ float t0[32][33], t1[32][33];
    const int b = blockIdx.z, p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    for (int j = ty; j < 32; j += 8) {
        const int co = c0 + j, p = p0 + tx;
        if (co < g.fo && p < g.woho) {
            const long i = ((long)b * g.fo + co) * g.woho + p;
            t0[j][tx] = __ldg(d0 + i);
            t1[j][tx] = __ldg(d1 + i);
        }
    }
    __syncthreads();
    for (int j = ty; j < 32; j += 8) {
        const int p = p0 + j, co = c0 + tx;
        if (co < g.fo && p < g.woho) {
            const long i = ((long)b * g.woho + p) * g.fo + co;
            o0[i] = t0[tx][j];
            o1[i] = t1[tx][j];
        }
    }
}

// dmu_a[b][ci][y][x] = J * sum over taps (ky, kx) whose output pixel ((y + off - ky) / s, (x + off - kx) / s) exists of
// C[b][(ci, ky, kx)][that pixel]; the variance with J * J. One thread per input element, x fastest.
__global__ void __launch_bounds__(256) col2im_kernel(const float *__restrict__ c0, const float *__restrict__ c1,
                                                     const float *__restrict__ jcb, G g, float *__restrict__ o0,
                                                     float *__restrict__ o1) {
    const long total = (long)g.B * g.fi * g.wihi;
    for (long t = (long)blockIdx.x * 256 + threadIdx.x; t < total; t += (long)gridDim.x * 256) {
        // t < 2^31 (checked at the entry points): 32-bit divisions
        const unsigned n = (unsigned)t / (unsigned)g.wihi;  // b * fi + ci
        const int q = (int)((unsigned)t - n * (unsigned)g.wihi);
        const int y = q / g.wi, x = q - y * g.wi;
        float a0 = 0.f, a1 = 0.f;
        // output rows / columns whose window contains the pixel: oy * s - off <= y <= oy * s - off + k - 1
        const int oy_lo = max(0, (y + g.off - g.k + g.stride) / g.stride), oy_hi = min(g.ho - 1, (y + g.off) / g.stride);
        const int ox_lo = max(0, (x + g.off - g.k + g.stride) / g.stride), ox_hi = min(g.wo - 1, (x + g.off) / g.stride);
        for (int oy = oy_lo; oy <= oy_hi; oy++) {
            const int ky = y + g.off - oy * g.stride;
            for (int ox = ox_lo; ox <= ox_hi; ox++) {
                const int kx = x + g.off - ox * g.stride;
                const long i = ((long)n * g.k2 + ky * g.k + kx) * g.woho + oy * g.wo + ox;
                a0 += __ldg(c0 + i);
                a1 += __ldg(c1 + i);
            }
        }
        const float j = jcb ? __ldg(jcb + t) : 1.f;
        o0[t] = a0 * j;
        o1[t] = a1 * j * j;
    }
}

inline unsigned grid_for(long total) {
    long blocks = (total + 255) / 256;
    return (unsigned)(blocks < 148L * 32 ? blocks : 148L * 32);
}
inline int ok_or(cudaError_t e, const char *what) { return e == cudaSuccess ? TAGI_OK : cuda_fail(e, what); }

// The CTA-pair kernel can gather a Conv2d operand itself. Every column tile of a row block gathers the block's operand
// again, so this pays while the output is at most two tiles (256 columns) wide: measured on the ResNet-18 shapes,
// 64 / 128 channels gain 30 % against the gather pass through scratch memory, 256 channels are level, 512 channels lose
// 10-20 %. TAGI_B200_CONV_GATHER=explicit / implicit forces one of the two, for comparison.
inline int gather_mode() {
    static const int mode = [] {
        const char *e = getenv("TAGI_B200_CONV_GATHER");
        return !e ? 0 : std::string(e) == "explicit" ? 1 : std::string(e) == "implicit" ? 2 : std::string(e) == "patch" ? 3 : 0;
    }();
    return mode;
}
// The patch kernels (tagi_conv_patch.cu) read the A operand of a channel block as one TMA box and take precedence where
// they apply (stride 1, 16 | channels, 4 | image width) and pay; TAGI_B200_CONV_GATHER=patch also lifts the width rule
// below, =implicit selects the cp.async gather of the Linear pair kernel instead.
inline bool patch_ok(const tagi_conv2d_geom &cg, int pass, long rows, int cols, std::initializer_list<const void *> ptrs) {
    const int mode = gather_mode();
    if (mode == 1 || mode == 2 || rows < 256) return false;
    // measured on the ResNet-18 shapes: the patch kernels win on tiles of at most 64 columns (64-channel layers: forward
    // 0.52 -> 0.48 ms, state pass 0.64 -> 0.42 ms) and in the state pass of 128-column layers with many rows (layer2:
    // 0.293 -> 0.272 ms); the forward pass with 128 columns is faster with the cp.async gather of the Linear pair kernel
    // (0.256 against 0.335 ms)
    const int widest = pass == CONV_PASS_STATE && rows >= 32768 ? 128 : 64;
    if (mode != 3 && cols > widest) return false;
    return conv_pix_patch_supported(cg, pass, ptrs);
}
inline bool implicit_ok(const G &g, long rows, int cols) {
    const int mode = gather_mode();
    // (the kernel keeps one validity bit per tap in a 64-bit word, bit 63 reserved: kernels up to 7 x 7)
    if (mode == 1 || g.k > 7 || rows >= (1L << 31) || !linear_tc_pair_for((int)rows)) return false;
    return mode == 2 || cols <= 256;
}

// Launches the tiled gather when the kernel size has an instantiation; returns false when the caller should use the
// general kernel. C, H, W: source tensor; OH, OW: pixel grid of the rows.
template <int NSRC, bool FLIP>
bool launch_gather_tiled(const float *s0, const float *s1, int B, int C, int H, int W, int OH, int OW, int k, int stride,
                         int off, float *d0, float *d1, cudaStream_t st) {
    if (k != 2 && k != 3 && k != 6) return false;
    TileGeom g;
    g.B = B, g.C = C, g.H = H, g.W = W, g.OH = OH, g.OW = OW, g.stride = FLIP ? 1 : stride, g.off = off;
    // tiles of up to 128 pixels: the row cut into equal pieces of at most 32 pixels, as many rows as fit
    const int nx = (OW + 31) / 32;
    g.tx = (OW + nx - 1) / nx;
    g.ty = GATHER_PIX / g.tx < OH ? GATHER_PIX / g.tx : OH;
    g.Kc = C * k * k;
    g.ct = C < GATHER_CT ? C : GATHER_CT;
    auto smem_of = [&](int ty) {
        const int IH = (ty - 1) * g.stride + k, IW = (g.tx - 1) * g.stride + k;
        return (size_t)NSRC * g.ct * IH * IW * sizeof(float);
    };
    while (g.ty > 1 && smem_of(g.ty) > 40 * 1024) g.ty--;
    const size_t smem = smem_of(g.ty);
    if (smem > 40 * 1024 || (long)B * OH * OW >= (1L << 31)) return false;
    g.tiles_x = (OW + g.tx - 1) / g.tx, g.tiles_y = (OH + g.ty - 1) / g.ty;
    const dim3 grid((unsigned)((long)B * g.tiles_x * g.tiles_y), (unsigned)((C + GATHER_CT - 1) / GATHER_CT));
    // 16-byte stores when every CTA's column block starts and ends on a multiple of 4 columns
    const int k2 = k * k, last = C % GATHER_CT;
    const bool vec = g.Kc % 4 == 0 && (g.ct * k2) % 4 == 0 && (last * k2) % 4 == 0 && aligned16(d0) && (NSRC == 1 || aligned16(d1));
#define TAGI_GATHER_LAUNCH(KSV)                                                                       \
    do {                                                                                              \
        if (vec) gather_tiled_kernel<NSRC, KSV, FLIP, 4><<<grid, 256, smem, st>>>(s0, s1, g, d0, d1); \
        else gather_tiled_kernel<NSRC, KSV, FLIP, 1><<<grid, 256, smem, st>>>(s0, s1, g, d0, d1);     \
    } while (0)
    if (k == 3)
        TAGI_GATHER_LAUNCH(3);
    else if (k == 6)
        TAGI_GATHER_LAUNCH(6);
    else
        TAGI_GATHER_LAUNCH(2);
#undef TAGI_GATHER_LAUNCH
    return true;
}

}  // namespace

// Which Conv2d calls the tensor-core kernels take: 16-byte aligned tensors and every GEMM dimension a multiple of 4
// (TMA row pitches, vector stores), and enough work for 128-row tiles.
bool conv_tc_supported(const tagi_conv2d_geom &cg, int pass, std::initializer_list<const void *> ptrs) {
    const G g = geom_of(cg);
    // row pitches of the matrices a pass hands to TMA (16-byte multiples) and its vector stores
    bool ok = g.Kc % 4 == 0;                                                   // X and the weights [fo][Kc]
    if (pass == CONV_PASS_PARAM) ok = ok && g.fo % 4 == 0;                      // D [rows][fo]
    if (pass == CONV_PASS_STATE)
        ok = ok && g.fo % 4 == 0 && (g.stride > 1 || g.fi % 4 == 0);           // D / Z, regrouped weights [..][fi]
    if (!ok) return false;
    for (const void *p : ptrs)
        if (p && !aligned16(p)) return false;
    return true;
}
// enough work for 128-row tiles with a contraction and a width that fill an MMA
bool conv_tc_profitable(const tagi_conv2d_geom &cg, int pass) {
    const G g = geom_of(cg);
    if ((long)g.B * g.woho < 256 || g.fo < 32) return false;
    // the GEMM's width is fi for the stride-1 state pass and fi*k*k for every other pass
    return pass == CONV_PASS_STATE && g.stride == 1 ? g.fi >= 16 : g.Kc >= 64;
}

// Upper bound of the scratch any of the three passes of this geometry asks for on the tensor-core path
size_t conv_tc_workspace_bytes(const tagi_conv2d_geom &cg) {
    const G g = geom_of(cg);
    const size_t rows = (size_t)g.B * g.woho, rows_in = (size_t)g.B * g.wihi, w = (size_t)g.fo * g.Kc;
    const size_t fwd = 2 * rows * g.Kc + 2 * w;
    const size_t state = g.stride > 1 ? 2 * rows * g.fo + 2 * rows * g.Kc : 2 * rows_in * g.fo * g.k2 + w;
    const int slices = linear_bwd_param_tc_slices((int)rows, g.Kc, g.fo);
    const size_t param = rows * g.Kc + 2 * rows * g.fo + (size_t)2 * (slices > 1 ? slices : 1) * w;
    size_t m = fwd > state ? fwd : state;
    m = m > param ? m : param;
    return m * sizeof(float);
}

int conv2d_fwd_tc(const tagi_conv2d_geom &cg, const float *mu_w, const float *var_w, const float *mu_b,
                  const float *var_b, const float *mu_a, const float *var_a, float *mu_z, float *var_z,
                  cudaStream_t st, float *relu_jcb) {
    const G g = geom_of(cg);
    const long rows = (long)g.B * g.woho;
    if (patch_ok(cg, CONV_PASS_FWD, rows, g.fo, {mu_a, var_a}))
        return conv2d_fwd_patch(cg, mu_w, var_w, mu_b, var_b, mu_a, var_a, mu_z, var_z, st, relu_jcb);
    if (implicit_ok(g, rows, g.fo)) {
        // implicit GEMM: the kernel gathers the receptive fields itself while it stages its A tiles
        ConvGather ig{1, mu_a, var_a, g.fi, g.hi, g.wi, g.wo, g.woho, g.k, g.stride, g.off, +1, rows};
        return linear_fwd_tc(mu_w, var_w, mu_b, var_b, nullptr, nullptr, (int)rows, g.Kc, g.fo, mu_z, var_z, st, g.woho, &ig,
                             relu_jcb);
    }
    float *ws = nullptr;
    int rc = conv_scratch((size_t)2 * rows * g.Kc * sizeof(float), &ws, st);
    if (rc != TAGI_OK) return rc;
    float *x_mu = ws, *x_var = ws + rows * g.Kc;
    if (!launch_gather_tiled<2, false>(mu_a, var_a, g.B, g.fi, g.hi, g.wi, g.ho, g.wo, g.k, g.stride, g.off, x_mu, x_var, st))
        im2col_kernel<2><<<grid_for(rows * g.Kc), 256, 0, st>>>(mu_a, var_a, g, x_mu, x_var);
    if ((rc = ok_or(cudaGetLastError(), "im2col kernel launch")) != TAGI_OK) return rc;
    // rows = (image, output pixel), columns = output channels: exactly Linear's forward, written as [b][co][pixel]
    return linear_fwd_tc(mu_w, var_w, mu_b, var_b, x_mu, x_var, (int)rows, g.Kc, g.fo, mu_z, var_z, st, g.woho, nullptr,
                         relu_jcb);
}
bool conv2d_fwd_tc_fuses_relu(const tagi_conv2d_geom &cg) {
    const G g = geom_of(cg);
    const long rows = (long)g.B * g.woho;
    return rows < (1L << 31) && linear_tc_pair_for((int)rows);
}

int conv2d_bwd_state_tc(const tagi_conv2d_geom &cg, const float *mu_w, const float *jcb, const float *dmu_z,
                        const float *dvar_z, float *dmu_a, float *dvar_a, cudaStream_t st) {
    const G g = geom_of(cg);
    float *ws = nullptr;
    int rc;
    if (g.stride > 1) {
        const long rows = (long)g.B * g.woho;
        if ((rc = conv_scratch(((size_t)2 * rows * g.fo + (size_t)2 * rows * g.Kc) * sizeof(float), &ws, st)) != TAGI_OK)
            return rc;
        float *d_mu = ws, *d_var = d_mu + rows * g.fo, *c_mu = d_var + rows * g.fo, *c_var = c_mu + rows * g.Kc;
        dim3 grid((g.woho + 31) / 32, (g.fo + 31) / 32, g.B);
        delta_regroup_kernel<<<grid, 256, 0, st>>>(dmu_z, dvar_z, g, d_mu, d_var);
        if ((rc = ok_or(cudaGetLastError(), "delta_regroup_kernel launch")) != TAGI_OK) return rc;
        // Linear's state pass without a Jacobian: C[(b, p)][kc] = sum over co of D[(b, p)][co] * w[co][kc] (and w * w for
        // the variance), stored as [b][kc][p]
        rc = linear_bwd_state_tc(mu_w, nullptr, d_mu, d_var, (int)rows, g.Kc, g.fo, c_mu, c_var, st, g.woho);
        if (rc != TAGI_OK) return rc;
        col2im_kernel<<<grid_for((long)g.B * g.fi * g.wihi), 256, 0, st>>>(c_mu, c_var, jcb, g, dmu_a, dvar_a);
        return ok_or(cudaGetLastError(), "col2im_kernel launch");
    }
    const long rows = (long)g.B * g.wihi;
    const int kd = g.fo * g.k2;
    if (patch_ok(cg, CONV_PASS_STATE, rows, g.fi, {dmu_z, dvar_z}))
        return conv2d_bwd_state_patch(cg, mu_w, jcb, dmu_z, dvar_z, dmu_a, dvar_a, st);
    if (implicit_ok(g, rows, g.fi)) {
        float *w2i = nullptr;
        if ((rc = conv_scratch((size_t)g.fo * g.Kc * sizeof(float), &w2i, st)) != TAGI_OK) return rc;
        weight_regroup_kernel<<<grid_for((long)g.fo * g.Kc), 256, 0, st>>>(mu_w, g, w2i);
        if ((rc = ok_or(cudaGetLastError(), "weight_regroup_kernel launch")) != TAGI_OK) return rc;
        // implicit GEMM: row = input pixel, column (co, ky, kx) = delta at output pixel (y + off - ky, x + off - kx)
        ConvGather ig{1, dmu_z, dvar_z, g.fo, g.ho, g.wo, g.wi, g.wihi, g.k, 1, g.off, -1, rows};
        return linear_bwd_state_tc(w2i, jcb, nullptr, nullptr, (int)rows, g.fi, kd, dmu_a, dvar_a, st, g.wihi, &ig);
    }
    rc = conv_scratch(((size_t)2 * rows * kd + (size_t)g.fo * g.Kc) * sizeof(float), &ws, st);
    if (rc != TAGI_OK) return rc;
    float *z_mu = ws, *z_var = ws + rows * kd, *w2 = ws + 2 * rows * kd;
    if (!launch_gather_tiled<2, true>(dmu_z, dvar_z, g.B, g.fo, g.ho, g.wo, g.hi, g.wi, g.k, 1, g.off, z_mu, z_var, st))
        delta_gather_kernel<<<grid_for(rows * kd), 256, 0, st>>>(dmu_z, dvar_z, g, z_mu, z_var);
    if ((rc = ok_or(cudaGetLastError(), "delta gather kernel launch")) != TAGI_OK) return rc;
    weight_regroup_kernel<<<grid_for((long)g.fo * g.Kc), 256, 0, st>>>(mu_w, g, w2);
    if ((rc = ok_or(cudaGetLastError(), "weight_regroup_kernel launch")) != TAGI_OK) return rc;
    // Linear's state pass with "output features" = (co, tap) and "input features" = ci; Jacobian and outputs in
    // [b][ci][pixel]
    return linear_bwd_state_tc(w2, jcb, z_mu, z_var, (int)rows, g.fi, kd, dmu_a, dvar_a, st, g.wihi);
}

int conv2d_bwd_param_tc(const tagi_conv2d_geom &cg, const float *var_w, const float *mu_a, const float *dmu_z,
                        const float *dvar_z, float *dmu_w, float *dvar_w, cudaStream_t st) {
    const G g = geom_of(cg);
    const long rows = (long)g.B * g.woho;
    // small weight tensors with a long contraction (B * ho * wo): the contraction is cut into slices
    const int slices = linear_bwd_param_tc_slices((int)rows, g.Kc, g.fo);
    const size_t part = slices > 1 ? (size_t)2 * slices * g.fo * g.Kc : 0;
    float *ws = nullptr;
    int rc = conv_scratch(((size_t)rows * g.Kc + (size_t)2 * rows * g.fo + part) * sizeof(float), &ws, st);
    if (rc != TAGI_OK) return rc;
    float *x_mu = ws, *d_mu = ws + rows * g.Kc, *d_var = d_mu + rows * g.fo, *split_ws = d_var + rows * g.fo;
    if (!launch_gather_tiled<1, false>(mu_a, nullptr, g.B, g.fi, g.hi, g.wi, g.ho, g.wo, g.k, g.stride, g.off, x_mu, nullptr, st))
        im2col_kernel<1><<<grid_for(rows * g.Kc), 256, 0, st>>>(mu_a, nullptr, g, x_mu, nullptr);
    if ((rc = ok_or(cudaGetLastError(), "im2col kernel launch")) != TAGI_OK) return rc;
    dim3 grid((g.woho + 31) / 32, (g.fo + 31) / 32, g.B);
    delta_regroup_kernel<<<grid, 256, 0, st>>>(dmu_z, dvar_z, g, d_mu, d_var);
    if ((rc = ok_or(cudaGetLastError(), "delta_regroup_kernel launch")) != TAGI_OK) return rc;
    // Linear's parameter pass with batch = (image, output pixel): dmu_w[co][kc] = var_w * sum D[.][co] X[.][kc]
    return linear_bwd_param_tc(var_w, x_mu, d_mu, d_var, (int)rows, g.Kc, g.fo, dmu_w, dvar_w, st,
                               slices > 1 ? split_ws : nullptr, slices);
}

}  // namespace tagi
