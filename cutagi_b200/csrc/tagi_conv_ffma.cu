// TAGI Conv2d as implicit GEMM on the FP32 FFMA tile engine: the receptive-field gather is computed
// from the geometry while a tile is staged, so there are no index tables, no im2col buffer and no
// permuted copies of the Jacobian or of the deltas. Arithmetic follows the reference's CPU
// definitions (src/conv2d_layer.cpp:274-322, 363-403, 459-494, 538-556 of cuTAGI) with the
// receptive-field rule of src/indices.cpp:63-104, 163-194.
//
// GEMM views (rows x columns x contraction):
//   forward          fo x (B*ho*wo) x (fi*k*k)      A = weights,          B = gathered activations
//   state backward   fi x (B*hi*wi) x (fo*k*k)      A = gathered weights, B = gathered output deltas
//   parameter bwd    fo x (fi*k*k)  x (B*ho*wo)     A = output deltas,    B = gathered activations
// The columns are the memory-contiguous index of each output tensor.
#include <mutex>
#include <vector>

#include "tagi_common.h"
#include "tagi_ffma.cuh"

namespace tagi {
namespace {

struct Geom {
    int B, fi, hi, wi, fo, ho, wo, k, stride, off;
    int k2, Kc, woho, wihi;
};
Geom make_geom(const tagi_conv2d_geom &g) {
    Geom q;
    q.B = g.B, q.fi = g.fi, q.hi = g.hi, q.wi = g.wi, q.fo = g.fo, q.ho = g.ho, q.wo = g.wo, q.k = g.k;
    q.stride = g.stride;
    q.off = g.pad_type == 1 ? g.pad : 0;
    q.k2 = g.k * g.k, q.Kc = q.k2 * g.fi, q.woho = g.wo * g.ho, q.wihi = g.wi * g.hi;
    return q;
}

// Activations seen by output pixel n = (b, oy, ox) through tap kc = (ci, ky, kx); zero outside the image.
template <int D>
struct ActForOutputPixel {
    static constexpr int NSRC = DeriveTraits<D>::NSRC, NSM = DeriveTraits<D>::NSM, DER = D;
    const float *src0, *src1;
    Geom g;
    int rows, kdim;
    struct Ctx {
        long base;
        int y0, x0;
        bool ok;
    };
    __device__ __forceinline__ Ctx row_ctx(int n) const {
        const int b = n / g.woho, p = n - b * g.woho, oy = p / g.wo, ox = p - oy * g.wo;
        return {(long)b * g.fi * g.wihi, oy * g.stride - g.off, ox * g.stride - g.off, n < rows};
    }
    __device__ __forceinline__ void load(const Ctx &c, int kc, float (&v)[NSM]) const {
        float x0 = 0.f, x1 = 0.f;
        if (c.ok && kc < kdim) {
            const int ci = kc / g.k2, t = kc - ci * g.k2, ky = t / g.k, kx = t - ky * g.k;
            const int y = c.y0 + ky, x = c.x0 + kx;
            if ((unsigned)y < (unsigned)g.hi && (unsigned)x < (unsigned)g.wi) {
                const long i = c.base + (long)ci * g.wihi + y * g.wi + x;
                x0 = __ldg(src0 + i);
                if (NSRC == 2) x1 = __ldg(src1 + i);
            }
        }
        derive<D>(x0, x1, v);
    }
};

// Same gather with the roles swapped for the parameter pass: row i = (ci, ky, kx), contraction kk = (b, oy, ox).
template <int D>
struct ActForTap {
    static constexpr int NSRC = DeriveTraits<D>::NSRC, NSM = DeriveTraits<D>::NSM, DER = D;
    const float *src0, *src1;
    Geom g;
    int rows, kdim;
    struct Ctx {
        long base;
        int dy, dx;
        bool ok;
    };
    __device__ __forceinline__ Ctx row_ctx(int i) const {
        const int ci = i / g.k2, t = i - ci * g.k2, ky = t / g.k, kx = t - ky * g.k;
        return {(long)ci * g.wihi, ky - g.off, kx - g.off, i < rows};
    }
    __device__ __forceinline__ void load(const Ctx &c, int kk, float (&v)[NSM]) const {
        float x0 = 0.f, x1 = 0.f;
        if (c.ok && kk < kdim) {
            const int b = kk / g.woho, p = kk - b * g.woho, oy = p / g.wo, ox = p - oy * g.wo;
            const int y = oy * g.stride + c.dy, x = ox * g.stride + c.dx;
            if ((unsigned)y < (unsigned)g.hi && (unsigned)x < (unsigned)g.wi) {
                const long i = (long)b * g.fi * g.wihi + c.base + y * g.wi + x;
                x0 = __ldg(src0 + i);
                if (NSRC == 2) x1 = __ldg(src1 + i);
            }
        }
        derive<D>(x0, x1, v);
    }
};

// Weights seen from input channel ci through kk = (co, ky, kx): mu_w[co][ci][ky][kx].
template <int D>
struct WeightForInputChannel {
    static constexpr int NSRC = DeriveTraits<D>::NSRC, NSM = DeriveTraits<D>::NSM, DER = D;
    const float *src0, *src1;
    Geom g;
    int rows, kdim;
    struct Ctx {
        long base;
        bool ok;
    };
    __device__ __forceinline__ Ctx row_ctx(int ci) const { return {(long)ci * g.k2, ci < rows}; }
    __device__ __forceinline__ void load(const Ctx &c, int kk, float (&v)[NSM]) const {
        float x0 = 0.f, x1 = 0.f;
        if (c.ok && kk < kdim) {
            const int co = kk / g.k2, t = kk - co * g.k2;
            const long i = (long)co * g.Kc + c.base + t;
            x0 = __ldg(src0 + i);
            if (NSRC == 2) x1 = __ldg(src1 + i);
        }
        derive<D>(x0, x1, v);
    }
};

// Output deltas that input pixel n = (b, y, x) receives through kk = (co, ky, kx): the output pixel
// ((y + off - ky) / stride, (x + off - kx) / stride) when that division is exact and inside the output.
template <int D>
struct DeltaForInputPixel {
    static constexpr int NSRC = DeriveTraits<D>::NSRC, NSM = DeriveTraits<D>::NSM, DER = D;
    const float *src0, *src1;
    Geom g;
    int rows, kdim;
    struct Ctx {
        long base;
        int y, x;
        bool ok;
    };
    __device__ __forceinline__ Ctx row_ctx(int n) const {
        const int b = n / g.wihi, q = n - b * g.wihi, y = q / g.wi, x = q - y * g.wi;
        return {(long)b * g.fo * g.woho, y + g.off, x + g.off, n < rows};
    }
    __device__ __forceinline__ void load(const Ctx &c, int kk, float (&v)[NSM]) const {
        float x0 = 0.f, x1 = 0.f;
        if (c.ok && kk < kdim) {
            const int co = kk / g.k2, t = kk - co * g.k2, ky = t / g.k, kx = t - ky * g.k;
            const int ty = c.y - ky, tx = c.x - kx;
            if (ty >= 0 && tx >= 0) {
                const int oy = ty / g.stride, ox = tx / g.stride;
                if (oy * g.stride == ty && ox * g.stride == tx && oy < g.ho && ox < g.wo) {
                    const long i = c.base + (long)co * g.woho + oy * g.wo + ox;
                    x0 = __ldg(src0 + i);
                    if (NSRC == 2) x1 = __ldg(src1 + i);
                }
            }
        }
        derive<D>(x0, x1, v);
    }
};

// Output deltas of channel co over kk = (b, p): delta[b][co][p].
template <int D>
struct DeltaForChannel {
    static constexpr int NSRC = DeriveTraits<D>::NSRC, NSM = DeriveTraits<D>::NSM, DER = D;
    const float *src0, *src1;
    Geom g;
    int rows, kdim;
    struct Ctx {
        long base;
        bool ok;
    };
    __device__ __forceinline__ Ctx row_ctx(int co) const { return {(long)co * g.woho, co < rows}; }
    __device__ __forceinline__ void load(const Ctx &c, int kk, float (&v)[NSM]) const {
        float x0 = 0.f, x1 = 0.f;
        if (c.ok && kk < kdim) {
            const int b = kk / g.woho, p = kk - b * g.woho;
            const long i = (long)b * g.fo * g.woho + c.base + p;
            x0 = __ldg(src0 + i);
            if (NSRC == 2) x1 = __ldg(src1 + i);
        }
        derive<D>(x0, x1, v);
    }
};

// Output tensors [b][chan][pix] written from GEMM coordinates (m = chan, n = b * npix + pix).
// bias: out = c + bias[m] (forward). scale: out1 = c1 * s, out2 = c2 * s * s with s = scale[same index].
struct EpiChanPix {
    float *out1, *out2;
    const float *bias1, *bias2;  // forward, may be null
    const float *scale;          // state backward (Jacobian), may be null
    int nchan, npix;
    bool vec_ok;  // npix % 4 == 0 and 16-byte aligned bases: four consecutive n stay inside one image
    __device__ __forceinline__ long index(int m, int n) const {
        const int b = n / npix, p = n - b * npix;
        return ((long)b * nchan + m) * npix + p;
    }
    __device__ __forceinline__ void store(int m, int n, int, float c1, float c2) const {
        const long i = index(m, n);
        if (bias1) {
            c1 += __ldg(bias1 + m);
            c2 += __ldg(bias2 + m);
        }
        if (scale) {
            const float s = __ldg(scale + i);
            c1 *= s;
            c2 = c2 * s * s;
        }
        out1[i] = c1;
        out2[i] = c2;
    }
    __device__ __forceinline__ void store4(int m, int n, int, float4 c1, float4 c2) const {
        const long i = index(m, n);
        if (bias1) {
            const float b1 = __ldg(bias1 + m), b2 = __ldg(bias2 + m);
            c1.x += b1, c1.y += b1, c1.z += b1, c1.w += b1;
            c2.x += b2, c2.y += b2, c2.z += b2, c2.w += b2;
        }
        if (scale) {
            const float4 s = __ldg(reinterpret_cast<const float4 *>(scale + i));
            c1.x *= s.x, c1.y *= s.y, c1.z *= s.z, c1.w *= s.w;
            c2.x = c2.x * s.x * s.x, c2.y = c2.y * s.y * s.y, c2.z = c2.z * s.z * s.z, c2.w = c2.w * s.w * s.w;
        }
        __stcs(reinterpret_cast<float4 *>(out1 + i), c1);
        __stcs(reinterpret_cast<float4 *>(out2 + i), c2);
    }
};

// Sum of the split-K slices in slice order, then the var_w scaling of the parameter pass.
__global__ void __launch_bounds__(256) reduce_slices_scale_kernel(const float *__restrict__ part1,
                                                                  const float *__restrict__ part2,
                                                                  const float *__restrict__ scale, long n, int slices,
                                                                  float *__restrict__ out1,
                                                                  float *__restrict__ out2) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float a1 = 0.f, a2 = 0.f;
    for (int z = 0; z < slices; z++) {
        a1 += part1[(long)z * n + i];
        a2 += part2[(long)z * n + i];
    }
    const float s = __ldg(scale + i);
    out1[i] = a1 * s;
    out2[i] = a2 * s * s;
}

// Bias deltas: dmu_b[co] = var_b * sum over (b, pixel) of dmu_z[b][co][pixel], dvar_b likewise with var_b^2
// (src/conv2d_layer.cpp:538-556). HBM-bound: one pass over the deltas. Stage 1: block (co, s) sums the images
// b = s, s + S, ... of channel co (fixed order inside the block); stage 2: one thread per channel adds the S partial
// sums in order and scales. The result does not depend on scheduling.
__global__ void __launch_bounds__(256) conv_bias_partial_kernel(const float *__restrict__ dmu_z,
                                                                const float *__restrict__ dvar_z, int B, int fo,
                                                                int woho, int S, float2 *__restrict__ part) {
    __shared__ float s1[256], s2[256];
    const int co = blockIdx.x, sl = blockIdx.y;
    float a1 = 0.f, a2 = 0.f;
    for (int b = sl; b < B; b += S) {
        const long base = ((long)b * fo + co) * woho;
        for (int p = threadIdx.x; p < woho; p += 256) {
            a1 += __ldg(dmu_z + base + p);
            a2 += __ldg(dvar_z + base + p);
        }
    }
    s1[threadIdx.x] = a1;
    s2[threadIdx.x] = a2;
    __syncthreads();
    for (int w = 128; w > 0; w >>= 1) {
        if (threadIdx.x < w) {
            s1[threadIdx.x] += s1[threadIdx.x + w];
            s2[threadIdx.x] += s2[threadIdx.x + w];
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) part[(long)co * S + sl] = make_float2(s1[0], s2[0]);
}
__global__ void __launch_bounds__(128) conv_bias_final_kernel(const float *__restrict__ var_b,
                                                              const float2 *__restrict__ part, int fo, int S,
                                                              float *__restrict__ dmu_b, float *__restrict__ dvar_b) {
    const int co = blockIdx.x * 128 + threadIdx.x;
    if (co >= fo) return;
    float a1 = 0.f, a2 = 0.f;
    for (int s = 0; s < S; s++) {
        const float2 v = part[(long)co * S + s];
        a1 += v.x;
        a2 += v.y;
    }
    const float vb = __ldg(var_b + co);
    dmu_b[co] = a1 * vb;
    dvar_b[co] = a2 * vb * vb;
}

inline int done(cudaError_t e, const char *what) { return e == cudaSuccess ? TAGI_OK : cuda_fail(e, what); }

}  // namespace

int conv2d_fwd_ffma(const tagi_conv2d_geom &cg, const float *mu_w, const float *var_w, const float *mu_b,
                    const float *var_b, const float *mu_a, const float *var_a, float *mu_z, float *var_z,
                    cudaStream_t st) {
    const Geom g = make_geom(cg);
    const int M = g.fo, N = g.B * g.woho, Kd = g.Kc;
    StridedOperand<DER_MEAN_VAR_W> W{mu_w, var_w, (long)g.Kc, 1, g.fo, g.Kc};
    ActForOutputPixel<DER_MEAN_VAR_ACT> X{mu_a, var_a, g, N, Kd};
    EpiChanPix epi{mu_z, var_z, mu_b, var_b, nullptr, g.fo, g.woho,
                   g.woho % 4 == 0 && aligned16(mu_z) && aligned16(var_z)};
    return done(dispatch_ffma<decltype(W), decltype(X), EpiChanPix, LOAD_K_VEC4, LOAD_K_SCALAR, LOAD_R_SCALAR,
                              LOAD_R_SCALAR>(W, X, epi, M, N, Kd, g.Kc % 4 == 0 && aligned16(mu_w) && aligned16(var_w),
                                             false, st),
                "conv2d forward launch");
}

int conv2d_bwd_state_ffma(const tagi_conv2d_geom &cg, const float *mu_w, const float *jcb, const float *dmu_z,
                          const float *dvar_z, float *dmu_a, float *dvar_a, cudaStream_t st) {
    const Geom g = make_geom(cg);
    const int M = g.fi, N = g.B * g.wihi, Kd = g.fo * g.k2;
    WeightForInputChannel<DER_SQUARE> W{mu_w, nullptr, g, g.fi, Kd};
    DeltaForInputPixel<DER_PAIR> D{dmu_z, dvar_z, g, N, Kd};
    EpiChanPix epi{dmu_a, dvar_a, nullptr, nullptr, jcb, g.fi, g.wihi,
                   g.wihi % 4 == 0 && aligned16(dmu_a) && aligned16(dvar_a) && (!jcb || aligned16(jcb))};
    return done(dispatch_ffma<decltype(W), decltype(D), EpiChanPix, LOAD_K_SCALAR, LOAD_K_SCALAR, LOAD_R_SCALAR,
                              LOAD_R_SCALAR>(W, D, epi, M, N, Kd, false, false, st),
                "conv2d state backward launch");
}

// Scratch of the Conv2d implementations (split-contraction partial sums here, regrouped weights and gathered matrices
// in the tensor-core path): one grow-only block per device, owned by the library. Calls that use it are ordered by the
// stream they run on; calls on different streams of one device that both need scratch must not overlap.
// A block that has been handed out is never freed while the library may still be used: when a larger one is needed the
// old block is retired (kept until tagi_release_scratch), because kernels already launched and CUDA graphs already
// captured may still hold its address.
namespace {
struct Scratch {
    float *ptr = nullptr;
    size_t bytes = 0;
    std::vector<float *> retired;
};
Scratch g_scratch[64];
std::mutex g_scratch_mu;

}  // namespace

// The partial sums live in a small array of their own in the library image (8 bytes x channels x 64 slices at most), so
// the pass needs no scratch from the shared block and may follow any other pass on the same stream.
constexpr int kBiasSlices = 64, kBiasMaxChannels = 4096;
static __device__ float2 g_bias_part[kBiasSlices * kBiasMaxChannels];

int conv_bias_delta(const tagi_conv2d_geom &cg, const float *var_b, const float *dmu_z, const float *dvar_z,
                    float *dmu_b, float *dvar_b, cudaStream_t st) {
    if (cg.fo > kBiasMaxChannels) return fail(TAGI_ERR_UNSUPPORTED, "bias deltas: more than 4096 output channels");
    static float2 *part[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= 64) return fail(TAGI_ERR_UNSUPPORTED, "device index out of range");
    {
        std::lock_guard<std::mutex> lk(g_scratch_mu);
        if (!part[dev]) {
            e = cudaGetSymbolAddress(reinterpret_cast<void **>(&part[dev]), g_bias_part);
            if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(bias partial sums)");
        }
    }
    const int S = cg.B < kBiasSlices ? cg.B : kBiasSlices;
    conv_bias_partial_kernel<<<dim3(cg.fo, S), 256, 0, st>>>(dmu_z, dvar_z, cg.B, cg.fo, cg.ho * cg.wo, S, part[dev]);
    if (cudaGetLastError() != cudaSuccess) return done(cudaGetLastError(), "conv_bias_partial_kernel launch");
    conv_bias_final_kernel<<<(cg.fo + 127) / 128, 128, 0, st>>>(var_b, part[dev], cg.fo, S, dmu_b, dvar_b);
    return done(cudaGetLastError(), "conv_bias_final_kernel launch");
}

int conv_scratch(size_t bytes, float **out, cudaStream_t st) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= 64) return fail(TAGI_ERR_UNSUPPORTED, "device index out of range");
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    Scratch &s = g_scratch[dev];
    if (s.bytes < bytes) {
        // no allocation while the caller's stream is being captured: it would break the capture
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(st, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
            return fail(TAGI_ERR_UNSUPPORTED,
                        "Conv2d scratch of " + std::to_string(bytes) + " bytes is needed while the stream is being captured (" +
                            std::to_string(s.bytes) + " reserved): call tagi_reserve_scratch before the capture");
        const size_t want = bytes + bytes / 2;
        float *fresh = nullptr;
        e = cudaMalloc(&fresh, want);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(Conv2d scratch)");
        if (s.ptr) s.retired.push_back(s.ptr);
        s.ptr = fresh;
        s.bytes = want;
    }
    *out = s.ptr;
    return TAGI_OK;
}

int reserve_scratch(size_t bytes) {
    float *p = nullptr;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= 64) return fail(TAGI_ERR_UNSUPPORTED, "device index out of range");
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    Scratch &s = g_scratch[dev];
    if (s.bytes >= bytes) return TAGI_OK;
    e = cudaMalloc(&p, bytes);   // exactly what was asked for: the caller has sized it
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(Conv2d scratch)");
    if (s.ptr) s.retired.push_back(s.ptr);
    s.ptr = p;
    s.bytes = bytes;
    return TAGI_OK;
}

size_t scratch_bytes() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    return g_scratch[dev].bytes;
}

int release_scratch() {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= 64) return fail(TAGI_ERR_UNSUPPORTED, "device index out of range");
    e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceSynchronize");
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    Scratch &s = g_scratch[dev];
    for (float *p : s.retired) cudaFree(p);
    s.retired.clear();
    if (s.ptr) cudaFree(s.ptr);
    s.ptr = nullptr;
    s.bytes = 0;
    return TAGI_OK;
}

// Scratch of the FFMA parameter pass (partial sums of the split contraction), same slicing rule as below
size_t conv_ffma_workspace_bytes(const tagi_conv2d_geom &cg) {
    const Geom g = make_geom(cg);
    const int M = g.fo, N = g.Kc, Kd = g.B * g.woho;
    const int tm = M >= 128 && N >= 128 ? 128 : 64;
    const long tiles = (long)((M + tm - 1) / tm) * ((N + tm - 1) / tm);
    long splits = (2 * 148 + tiles - 1) / tiles;
    const long max_splits = (Kd + 255) / 256;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    return (size_t)2 * splits * M * N * sizeof(float);
}

int conv2d_bwd_param_ffma(const tagi_conv2d_geom &cg, const float *var_w, const float *var_b, const float *mu_a,
                          const float *dmu_z, const float *dvar_z, float *dmu_w, float *dvar_w, float *dmu_b,
                          float *dvar_b, cudaStream_t st) {
    const Geom g = make_geom(cg);
    const int M = g.fo, N = g.Kc, Kd = g.B * g.woho;
    DeltaForChannel<DER_PAIR> D{dmu_z, dvar_z, g, g.fo, Kd};
    ActForTap<DER_SQUARE> X{mu_a, nullptr, g, g.Kc, Kd};

    // The output (fo x fi*k*k) is small and the contraction (B*ho*wo) long: slice the contraction so that
    // about two CTAs per SM are in flight.
    const bool big = M >= 128 && N >= 128;
    const int tm = big ? 128 : 64;
    const long tiles = (long)((M + tm - 1) / tm) * ((N + tm - 1) / tm);
    int splits = (int)((2 * 148 + tiles - 1) / tiles);
    const int max_splits = (Kd + 255) / 256;  // keep at least 256 contraction steps per slice
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;

    int rc;
    if (splits == 1) {
        EpiRowScale epi{dmu_w, dvar_w, var_w, (long)N,
                        N % 4 == 0 && aligned16(dmu_w) && aligned16(dvar_w) && aligned16(var_w)};
        rc = done(dispatch_ffma<decltype(D), decltype(X), EpiRowScale, LOAD_K_SCALAR, LOAD_K_SCALAR, LOAD_K_SCALAR,
                                LOAD_K_SCALAR>(D, X, epi, M, N, Kd, false, false, st),
                  "conv2d parameter backward launch");
    } else {
        const long slice = (long)M * N;
        float *ws = nullptr;
        rc = conv_scratch((size_t)2 * splits * slice * sizeof(float), &ws, st);
        if (rc != TAGI_OK) return rc;
        EpiPartial epi{ws, ws + (long)splits * slice, (long)N, slice, N % 4 == 0};
        // the kernel may use fewer slices than asked for (slice length is rounded up); it reports through the grid,
        // so recompute the same rounding here
        const int bk = use_large_tile(M, N, splits) ? TileL::BK : TileS::BK;
        const int k_chunk = ((Kd + splits - 1) / splits + bk - 1) / bk * bk;
        const int slices = (Kd + k_chunk - 1) / k_chunk;
        rc = done(dispatch_ffma<decltype(D), decltype(X), EpiPartial, LOAD_K_SCALAR, LOAD_K_SCALAR, LOAD_K_SCALAR,
                                LOAD_K_SCALAR>(D, X, epi, M, N, Kd, false, false, st, splits),
                  "conv2d parameter backward launch");
        if (rc != TAGI_OK) return rc;
        reduce_slices_scale_kernel<<<(unsigned)((slice + 255) / 256), 256, 0, st>>>(
            ws, ws + (long)splits * slice, var_w, slice, slices, dmu_w, dvar_w);
        rc = done(cudaGetLastError(), "reduce_slices_scale_kernel launch");
    }
    if (rc != TAGI_OK) return rc;
    if (cg.has_bias) rc = conv_bias_delta(cg, var_b, dmu_z, dvar_z, dmu_b, dvar_b, st);
    return rc;
}

// ---------------------------------------------------------------------------------------------------------
// Parameter pass with statically reserved scratch (entry point tagi_conv2d_bwd_param_noalloc)
// ---------------------------------------------------------------------------------------------------------
// Some hosts of this library must not allocate device memory while they run: trainers that hand the whole GPU to their
// own pool at start-up (a later cudaMalloc fails or fragments that pool), services whose memory budget is fixed when
// they are admitted to a shared GPU, and code that runs while a thread of the process is capturing a stream in the
// global capture mode, where cudaMalloc is not a permitted call. For them the split-contraction scratch lives in the
// array below, which is part of the library image: every GPU that loads the library holds these 16 MiB until the
// process exits, whether or not this entry point is ever called.
//
// In host code the array's name is only a handle for the runtime, not a device address; the address a kernel can use
// comes from cudaGetSymbolAddress, asked once per device with that device current.
constexpr size_t kStaticScratchFloats = (size_t)4 << 20;  // 4 Mi floats = 16 MiB
constexpr long kNoAllocMaxWeights = (long)(kStaticScratchFloats / 4);  // two slices of both partial tensors must fit
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

namespace {
float *g_static_scratch_addr[64] = {};
std::mutex g_static_scratch_mu;

// Device address of g_static_scratch on the current device. The first call on a device asks the runtime for it.
int static_scratch(float **out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= 64) return fail(TAGI_ERR_UNSUPPORTED, "device index out of range");
    std::lock_guard<std::mutex> lk(g_static_scratch_mu);
    if (!g_static_scratch_addr[dev]) {
        float *ptr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_static_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
        g_static_scratch_addr[dev] = ptr;
    }
    *out = g_static_scratch_addr[dev];
    return TAGI_OK;
}
}  // namespace

int conv2d_bwd_param_noalloc(const tagi_conv2d_geom &cg, const float *var_w, const float *var_b, const float *mu_a,
                             const float *dmu_z, const float *dvar_z, float *dmu_w, float *dvar_w, float *dmu_b,
                             float *dvar_b, cudaStream_t st) {
    const Geom g = make_geom(cg);
    const int M = g.fo, N = g.Kc, Kd = g.B * g.woho;
    const long slice = (long)M * N;
    if (slice > kNoAllocMaxWeights)
        return fail(TAGI_ERR_UNSUPPORTED,
                    "tagi_conv2d_bwd_param_noalloc: weight tensor of " + std::to_string(slice) +
                        " elements exceeds the limit of " + std::to_string(kNoAllocMaxWeights) +
                        " (16 MiB of static scratch); use tagi_conv2d_bwd_param");
    DeltaForChannel<DER_PAIR> D{dmu_z, dvar_z, g, g.fo, Kd};
    ActForTap<DER_SQUARE> X{mu_a, nullptr, g, g.Kc, Kd};

    // same slicing rule as the allocating entry point, then as many slices as the static scratch holds
    const bool big = M >= 128 && N >= 128;
    const int tm = big ? 128 : 64;
    const long tiles = (long)((M + tm - 1) / tm) * ((N + tm - 1) / tm);
    int splits = (int)((2 * 148 + tiles - 1) / tiles);
    const int max_splits = (Kd + 255) / 256;
    if (splits > max_splits) splits = max_splits;
    const long fit = (long)(kStaticScratchFloats / (2 * (size_t)slice));
    if (splits > fit) splits = (int)fit;
    if (splits < 1) splits = 1;

    int rc;
    if (splits == 1) {
        EpiRowScale epi{dmu_w, dvar_w, var_w, (long)N,
                        N % 4 == 0 && aligned16(dmu_w) && aligned16(dvar_w) && aligned16(var_w)};
        rc = done(dispatch_ffma<decltype(D), decltype(X), EpiRowScale, LOAD_K_SCALAR, LOAD_K_SCALAR, LOAD_K_SCALAR,
                                LOAD_K_SCALAR>(D, X, epi, M, N, Kd, false, false, st),
                  "conv2d parameter backward launch");
    } else {
        float *ws = nullptr;
        rc = static_scratch(&ws);
        if (rc != TAGI_OK) return rc;
        // every slice overwrites its whole M x N part of both partial tensors, so nothing has to start at zero
        EpiPartial epi{ws, ws + (long)splits * slice, (long)N, slice, N % 4 == 0};
        const int bk = use_large_tile(M, N, splits) ? TileL::BK : TileS::BK;
        const int k_chunk = ((Kd + splits - 1) / splits + bk - 1) / bk * bk;
        const int slices = (Kd + k_chunk - 1) / k_chunk;
        rc = done(dispatch_ffma<decltype(D), decltype(X), EpiPartial, LOAD_K_SCALAR, LOAD_K_SCALAR, LOAD_K_SCALAR,
                                LOAD_K_SCALAR>(D, X, epi, M, N, Kd, false, false, st, splits),
                  "conv2d parameter backward launch");
        if (rc != TAGI_OK) return rc;
        reduce_slices_scale_kernel<<<(unsigned)((slice + 255) / 256), 256, 0, st>>>(
            ws, ws + (long)splits * slice, var_w, slice, slices, dmu_w, dvar_w);
        rc = done(cudaGetLastError(), "reduce_slices_scale_kernel launch");
    }
    if (rc != TAGI_OK) return rc;
    if (cg.has_bias) rc = conv_bias_delta(cg, var_b, dmu_z, dvar_z, dmu_b, dvar_b, st);
    return rc;
}

}  // namespace tagi
