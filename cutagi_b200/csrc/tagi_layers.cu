// The layers that sit between the Conv2d calls of the CNN / ResNet configurations: BatchNorm2d, AvgPool2d and the
// residual add. All of them are HBM-bound passes over [B][C][H*W] activations; each follows the reference's CPU
// definition (cited at the kernels), the reference's CUDA counterparts are cited at the entry points.
//
// BatchNorm2d statistics and parameter deltas are per-channel sums over B * H * W elements. A channel's elements are
// cut into slices of 4096 (in the reference's (image, pixel) order); one CTA reduces a slice, and a second kernel
// merges the slices of a channel in slice order, so results do not depend on scheduling. The variance is merged from
// per-slice (count, mean, M2) triples (Chan et al.), which keeps the accuracy of the reference's two-pass formula
// while the data is read once.
#include "tagi_common.h"

#include <type_traits>

namespace tagi {
namespace {

constexpr int BLOCK = 256;
constexpr int PER_THREAD = 16;
constexpr int SLICE = BLOCK * PER_THREAD;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// Sum over the CTA, result in every thread. `red` holds one float per warp; two barriers per call.
__device__ __forceinline__ float block_sum(float v, float *red) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < BLOCK / 32; w++) t += red[w];
    return t;
}

// Address of element i (0 <= i < B * wihi, (image, pixel) order) of channel c
__device__ __forceinline__ long chan_elem(long i, int c, int C, int wihi) {
    const unsigned b = (unsigned)i / (unsigned)wihi;  // i < B * wihi < 2^31 (checked at the entry points): 32-bit division
    return ((long)b * C + c) * wihi + ((unsigned)i - b * (unsigned)wihi);
}

// src/batchnorm_layer.cpp:127-168. Partial of slice s of channel c: (count, mean, M2, sum of var_a).
// VEC = 4: H*W is a multiple of 4 and the tensors are 16-byte aligned (16-byte loads, see bn2d_bwd_kernel).
template <int VEC>
__global__ void __launch_bounds__(BLOCK) bn2d_stats_partial_kernel(const float *__restrict__ mu_a,
                                                                   const float *__restrict__ var_a, int C, int wihi,
                                                                   long n, float4 *__restrict__ part) {
    __shared__ float red[BLOCK / 32];
    const int c = blockIdx.y;
    const long i0 = (long)blockIdx.x * SLICE;
    const int cnt = (int)min((long)SLICE, n - i0);
    float x[PER_THREAD];
    float sm = 0.f, sv = 0.f;
#pragma unroll
    for (int e = 0; e < PER_THREAD / VEC; e++) {
        const int j = (threadIdx.x + e * BLOCK) * VEC;
#pragma unroll
        for (int v = 0; v < VEC; v++) x[e * VEC + v] = 0.f;
        if (j < cnt) {  // cnt is a multiple of VEC: a group of VEC elements is inside the slice or outside it
            const long a = chan_elem(i0 + j, c, C, wihi);
            if (VEC == 4) {
                const float4 m = __ldg(reinterpret_cast<const float4 *>(mu_a + a));
                const float4 v = __ldg(reinterpret_cast<const float4 *>(var_a + a));
                x[e * 4] = m.x, x[e * 4 + 1] = m.y, x[e * 4 + 2] = m.z, x[e * 4 + 3] = m.w;
                sm += (m.x + m.y) + (m.z + m.w);
                sv += (v.x + v.y) + (v.z + v.w);
            } else {
                x[e] = __ldg(mu_a + a);
                sm += x[e];
                sv += __ldg(var_a + a);
            }
        }
    }
    sm = block_sum(sm, red);
    sv = block_sum(sv, red);
    const float mean = sm / cnt;
    float m2 = 0.f;
#pragma unroll
    for (int e = 0; e < PER_THREAD / VEC; e++)
        if ((threadIdx.x + e * BLOCK) * VEC < cnt) {
#pragma unroll
            for (int v = 0; v < VEC; v++) m2 += (x[e * VEC + v] - mean) * (x[e * VEC + v] - mean);
        }
    m2 = block_sum(m2, red);
    if (threadIdx.x == 0) part[(long)c * gridDim.x + blockIdx.x] = make_float4((float)cnt, mean, m2, sv);
}

// Merge of a channel's slices, then the running averages (src/batchnorm_layer.cpp:15-26)
__global__ void bn2d_stats_final_kernel(const float4 *__restrict__ part, int slices, long n, float momentum,
                                        float *__restrict__ mean_out, float *__restrict__ var_out,
                                        float *__restrict__ mu_ra, float *__restrict__ var_ra, int C) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const float4 *p = part + (long)c * slices;
    double s = 0.0;
    for (int i = 0; i < slices; i++) s += (double)p[i].x * p[i].y;
    const double mean = s / (double)n;
    double m2 = 0.0, sv = 0.0;
    for (int i = 0; i < slices; i++) {
        const double d = (double)p[i].y - mean;
        m2 += (double)p[i].z + (double)p[i].x * d * d;
        sv += (double)p[i].w;
    }
    const float m = (float)mean, v = (float)((m2 + sv) / (double)(n - 1));
    mean_out[c] = m;
    var_out[c] = v;
    mu_ra[c] = mu_ra[c] * momentum + m * (1.f - momentum);
    var_ra[c] = var_ra[c] * momentum + v * (1.f - momentum);
}

struct BnChan {
    float inv, mean, w, w2v, vw, mb, vb;  // 1/sqrt(var+eps), mean, mu_w, mu_w^2 + var_w, var_w, mu_b, var_b
};
__device__ __forceinline__ BnChan bn_chan(int c, float eps, const float *mu_w, const float *var_w, const float *mu_b,
                                          const float *var_b, const float *mean, const float *var) {
    BnChan k;
    k.inv = 1.0f / sqrtf(__ldg(var + c) + eps);
    k.mean = __ldg(mean + c);
    k.w = __ldg(mu_w + c);
    k.vw = __ldg(var_w + c);
    k.w2v = k.w * k.w + k.vw;
    k.mb = mu_b ? __ldg(mu_b + c) : 0.f;
    k.vb = var_b ? __ldg(var_b + c) : 0.f;
    return k;
}
__device__ __forceinline__ void bn_apply(const BnChan &k, float a, float va, float &z, float &vz) {
    const float t = a - k.mean;
    z = k.inv * t * k.w + k.mb;
    vz = k.inv * k.inv * (va * k.w2v + k.vw * t * t) + k.vb;
}

// src/batchnorm_layer.cpp:170-206. VEC = 4: H*W is a multiple of 4, so four consecutive elements share a channel.
template <int VEC>
__global__ void __launch_bounds__(BLOCK) bn2d_apply_kernel(const float *__restrict__ mu_w, const float *__restrict__ var_w,
                                                           const float *__restrict__ mu_b, const float *__restrict__ var_b,
                                                           const float *__restrict__ mu_a, const float *__restrict__ var_a,
                                                           const float *__restrict__ mean, const float *__restrict__ var,
                                                           float eps, int C, int wihi, long total,
                                                           float *__restrict__ mu_z, float *__restrict__ var_z) {
    const long t = ((long)blockIdx.x * BLOCK + threadIdx.x) * VEC;
    if (t >= total) return;
    const int c = (int)((t / wihi) % C);
    const BnChan k = bn_chan(c, eps, mu_w, var_w, mu_b, var_b, mean, var);
    if (VEC == 4) {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(mu_a + t));
        const float4 v = __ldg(reinterpret_cast<const float4 *>(var_a + t));
        float4 z, vz;
        bn_apply(k, a.x, v.x, z.x, vz.x);
        bn_apply(k, a.y, v.y, z.y, vz.y);
        bn_apply(k, a.z, v.z, z.z, vz.z);
        bn_apply(k, a.w, v.w, z.w, vz.w);
        *reinterpret_cast<float4 *>(mu_z + t) = z;
        *reinterpret_cast<float4 *>(var_z + t) = vz;
    } else {
        float z, vz;
        bn_apply(k, __ldg(mu_a + t), __ldg(var_a + t), z, vz);
        mu_z[t] = z;
        var_z[t] = vz;
    }
}

// State deltas (src/batchnorm_layer.cpp:233-255) and the per-slice sums of the parameter deltas (:307-357) in one
// pass over the saved input, the Jacobian and the incoming deltas.
// Partial of slice s of channel c: (sum t * dmu_o, sum t * t * dvar_o, sum dmu_o, sum dvar_o), t = inv * (mu_a - mean) * var_w.
// VEC = 4: H*W is a multiple of 4 and the tensors are 16-byte aligned, so every group of four consecutive elements of a
// channel lies in one image plane and moves as one 16-byte access.
template <int VEC>
__global__ void __launch_bounds__(BLOCK) bn2d_bwd_kernel(const float *__restrict__ mu_w, const float *__restrict__ var_w,
                                                         const float *__restrict__ mu_a, const float *__restrict__ jcb,
                                                         const float *__restrict__ mean, const float *__restrict__ var,
                                                         const float *__restrict__ dmu_o, const float *__restrict__ dvar_o,
                                                         float eps, int C, int wihi, long n, int state_update,
                                                         float *__restrict__ dmu, float *__restrict__ dvar,
                                                         float4 *__restrict__ part) {
    __shared__ float red[BLOCK / 32];
    const int c = blockIdx.y;
    const long i0 = (long)blockIdx.x * SLICE;
    const int cnt = (int)min((long)SLICE, n - i0);
    const float inv = 1.0f / sqrtf(__ldg(var + c) + eps), m = __ldg(mean + c), w = __ldg(mu_w + c), vw = __ldg(var_w + c);
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    auto one = [&](float a_, float j_, float dm, float dv, float &o1, float &o2) {
        const float t = inv * (a_ - m) * vw;
        s0 += t * dm;
        s1 += t * dv * t;
        s2 += dm;
        s3 += dv;
        const float u = inv * w * j_;
        o1 = u * dm;
        o2 = u * dv * u;
    };
#pragma unroll 4
    for (int e = 0; e < PER_THREAD / VEC; e++) {
        const int j = (threadIdx.x + e * BLOCK) * VEC;
        if (j < cnt) {
            const long a = chan_elem(i0 + j, c, C, wihi);
            if (VEC == 4) {
                const float4 dm = __ldg(reinterpret_cast<const float4 *>(dmu_o + a));
                const float4 dv = __ldg(reinterpret_cast<const float4 *>(dvar_o + a));
                const float4 x = __ldg(reinterpret_cast<const float4 *>(mu_a + a));
                const float4 jj = jcb ? __ldg(reinterpret_cast<const float4 *>(jcb + a)) : make_float4(1.f, 1.f, 1.f, 1.f);
                float4 o1, o2;
                one(x.x, jj.x, dm.x, dv.x, o1.x, o2.x);
                one(x.y, jj.y, dm.y, dv.y, o1.y, o2.y);
                one(x.z, jj.z, dm.z, dv.z, o1.z, o2.z);
                one(x.w, jj.w, dm.w, dv.w, o1.w, o2.w);
                if (state_update) {
                    *reinterpret_cast<float4 *>(dmu + a) = o1;
                    *reinterpret_cast<float4 *>(dvar + a) = o2;
                }
            } else {
                float o1, o2;
                one(__ldg(mu_a + a), jcb ? __ldg(jcb + a) : 1.f, __ldg(dmu_o + a), __ldg(dvar_o + a), o1, o2);
                if (state_update) {
                    dmu[a] = o1;
                    dvar[a] = o2;
                }
            }
        }
    }
    s0 = block_sum(s0, red);
    s1 = block_sum(s1, red);
    s2 = block_sum(s2, red);
    s3 = block_sum(s3, red);
    if (threadIdx.x == 0) part[(long)c * gridDim.x + blockIdx.x] = make_float4(s0, s1, s2, s3);
}

__global__ void bn2d_bwd_final_kernel(const float4 *__restrict__ part, int slices, const float *__restrict__ var_b, int C,
                                      float *__restrict__ dmu_w, float *__restrict__ dvar_w, float *__restrict__ dmu_b,
                                      float *__restrict__ dvar_b) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const float4 *p = part + (long)c * slices;
    double s0 = 0, s1 = 0, s2 = 0, s3 = 0;
    for (int i = 0; i < slices; i++) s0 += p[i].x, s1 += p[i].y, s2 += p[i].z, s3 += p[i].w;
    dmu_w[c] = (float)s0;
    dvar_w[c] = (float)s1;
    if (var_b) {  // src/batchnorm_layer.cpp:334-357: each term scaled by var_b (mean) and var_b^2 (variance)
        const float vb = var_b[c];
        dmu_b[c] = vb * (float)s2;
        dvar_b[c] = vb * (float)s3 * vb;
    }
}

struct PoolGeom {
    int C, hi, wi, ho, wo, k, stride, off, overlap;
};

// src/pooling_layer.cpp:207-283: mean of the taps inside the image over k*k, variance over k^4; one thread per output
__global__ void __launch_bounds__(BLOCK) avgpool2d_fwd_kernel(const float *__restrict__ mu_a, const float *__restrict__ var_a,
                                                              PoolGeom g, long total, float *__restrict__ mu_z,
                                                              float *__restrict__ var_z) {
    const long t = (long)blockIdx.x * BLOCK + threadIdx.x;
    if (t >= total) return;
    // total < 2^31 (checked at the entry points): 32-bit divisions
    const unsigned woho = g.wo * g.ho, plane = (unsigned)t / woho;
    const int p = (int)((unsigned)t - plane * woho), oy = p / g.wo, ox = p - oy * g.wo;
    const float *a = mu_a + (size_t)plane * g.hi * g.wi, *v = var_a + (size_t)plane * g.hi * g.wi;
    float sm = 0.f, sv = 0.f;
    for (int ky = 0; ky < g.k; ky++) {
        const int y = oy * g.stride - g.off + ky;
        if ((unsigned)y >= (unsigned)g.hi) continue;
        for (int kx = 0; kx < g.k; kx++) {
            const int x = ox * g.stride - g.off + kx;
            if ((unsigned)x >= (unsigned)g.wi) continue;
            sm += __ldg(a + y * g.wi + x);
            sv += __ldg(v + y * g.wi + x);
        }
    }
    const int k2 = g.k * g.k;
    mu_z[t] = sm / k2;
    var_z[t] = sv / (k2 * k2);
}

// src/pooling_layer.cpp:285-375: each input pixel collects the deltas of the cells that contain it; one thread per VEC
// consecutive pixels of a row (VEC = 4: wi a multiple of 4 and 16-byte aligned tensors)
template <int VEC>
__global__ void __launch_bounds__(BLOCK) avgpool2d_bwd_kernel(const float *__restrict__ jcb, const float *__restrict__ dmu_o,
                                                              const float *__restrict__ dvar_o, PoolGeom g, unsigned items,
                                                              float *__restrict__ dmu, float *__restrict__ dvar) {
    const unsigned it = blockIdx.x * BLOCK + threadIdx.x;
    if (it >= items) return;
    const unsigned t = it * VEC, wihi = g.wi * g.hi, plane = t / wihi, q = t - plane * wihi;
    const int y = q / g.wi, x0 = q - y * g.wi;
    const float *dm = dmu_o + (size_t)plane * g.ho * g.wo, *dv = dvar_o + (size_t)plane * g.ho * g.wo;
    float sm[VEC], sv[VEC];
    if (!g.overlap) {  // k == stride: the cell of the pixel; k == image width (global pooling): the only cell
        const int oy = g.k == g.stride ? y / g.k : 0;
#pragma unroll
        for (int v = 0; v < VEC; v++) {
            const int ox = g.k == g.stride ? (x0 + v) / g.k : 0;
            const bool in = oy < g.ho && ox < g.wo;
            sm[v] = in ? __ldg(dm + oy * g.wo + ox) : 0.f;
            sv[v] = in ? __ldg(dv + oy * g.wo + ox) : 0.f;
        }
    } else {
        // cells whose window contains the pixel, in ascending order (the order of the reference's index table)
        const int oy_lo = max(0, (y + g.off - g.k + g.stride) / g.stride), oy_hi = min(g.ho - 1, (y + g.off) / g.stride);
        int lo[VEC], hi[VEC];
#pragma unroll
        for (int v = 0; v < VEC; v++) {
            const int x = x0 + v;
            lo[v] = max(0, (x + g.off - g.k + g.stride) / g.stride), hi[v] = min(g.wo - 1, (x + g.off) / g.stride);
            sm[v] = sv[v] = 0.f;
        }
        // every cell is loaded once for the VEC pixels; each pixel adds its own cells in the same ascending order.
        // MAXC: cells of a row that the VEC pixels share (3 for 3 x 3 windows at stride 2: the narrow variant)
        auto shared_cells = [&](auto maxc_tag) {
            constexpr int MAXC = decltype(maxc_tag)::value;
            for (int oy = oy_lo; oy <= oy_hi; oy++) {
                float cm[MAXC], cv[MAXC];
#pragma unroll
                for (int c = 0; c < MAXC; c++) {
                    const bool in = lo[0] + c <= hi[VEC - 1];
                    cm[c] = in ? __ldg(dm + oy * g.wo + lo[0] + c) : 0.f;
                    cv[c] = in ? __ldg(dv + oy * g.wo + lo[0] + c) : 0.f;
                }
#pragma unroll
                for (int v = 0; v < VEC; v++)
#pragma unroll
                    for (int c = 0; c < MAXC; c++)
                        if (lo[0] + c >= lo[v] && lo[0] + c <= hi[v]) sm[v] += cm[c], sv[v] += cv[c];
            }
        };
        const int span = hi[VEC - 1] - lo[0];
        if (VEC > 1 && span < 4) {
            shared_cells(std::integral_constant<int, 4>());
        } else if (VEC > 1 && span < 8) {
            shared_cells(std::integral_constant<int, 8>());
        } else {
#pragma unroll
            for (int v = 0; v < VEC; v++)
                for (int oy = oy_lo; oy <= oy_hi; oy++)
                    for (int ox = lo[v]; ox <= hi[v]; ox++) {
                        sm[v] += __ldg(dm + oy * g.wo + ox);
                        sv[v] += __ldg(dv + oy * g.wo + ox);
                    }
        }
    }
    const int k2 = g.k * g.k;
    if (VEC == 4) {
        const float4 j = jcb ? __ldg(reinterpret_cast<const float4 *>(jcb + t)) : make_float4(1.f, 1.f, 1.f, 1.f);
        *reinterpret_cast<float4 *>(dmu + t) = make_float4(sm[0] * j.x / k2, sm[1] * j.y / k2, sm[2] * j.z / k2, sm[3] * j.w / k2);
        const int k4 = k2 * k2;
        *reinterpret_cast<float4 *>(dvar + t) =
            make_float4(sv[0] * j.x * j.x / k4, sv[1] * j.y * j.y / k4, sv[2] * j.z * j.z / k4, sv[3] * j.w * j.w / k4);
    } else {
        const float j = jcb ? __ldg(jcb + t) : 1.f;
        dmu[t] = sm[0] * j / k2;
        dvar[t] = sv[0] * j * j / (k2 * k2);
    }
}

// src/resnet_block.cpp:8-31
__global__ void __launch_bounds__(BLOCK) add_shortcut_kernel(const float *__restrict__ mu_s, const float *__restrict__ var_s,
                                                             const float *__restrict__ jcb, size_t n, float *__restrict__ mu_a,
                                                             float *__restrict__ var_a) {
    const size_t i = (size_t)blockIdx.x * BLOCK + threadIdx.x;
    if (i >= n) return;
    const float j = jcb ? __ldg(jcb + i) : 1.f;
    mu_a[i] += __ldg(mu_s + i) * j;
    var_a[i] += __ldg(var_s + i) * j * j;
}

// four elements per thread with 16-byte accesses (n a multiple of 4, 16-byte aligned tensors)
__global__ void __launch_bounds__(BLOCK) add_shortcut_vec4_kernel(const float4 *__restrict__ mu_s, const float4 *__restrict__ var_s,
                                                                  const float4 *__restrict__ jcb, size_t n4,
                                                                  float4 *__restrict__ mu_a, float4 *__restrict__ var_a) {
    const size_t i = (size_t)blockIdx.x * BLOCK + threadIdx.x;
    if (i >= n4) return;
    const float4 j = jcb ? __ldg(jcb + i) : make_float4(1.f, 1.f, 1.f, 1.f);
    const float4 s = __ldg(mu_s + i), vs = __ldg(var_s + i);
    float4 a = mu_a[i], va = var_a[i];
    a.x += s.x * j.x, a.y += s.y * j.y, a.z += s.z * j.z, a.w += s.w * j.w;
    va.x += vs.x * j.x * j.x, va.y += vs.y * j.y * j.y, va.z += vs.z * j.z * j.z, va.w += vs.w * j.w * j.w;
    mu_a[i] = a;
    var_a[i] = va;
}

inline int launched(const char *what) {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? TAGI_OK : cuda_fail(e, what);
}

}  // namespace

int bn2d_fwd(int B, int C, int wihi, int training, float eps, float momentum, const float *mu_w, const float *var_w,
             const float *mu_b, const float *var_b, const float *mu_a, const float *var_a, float *mu_ra, float *var_ra,
             float *mu_batch, float *var_batch, float *mu_z, float *var_z, cudaStream_t st) {
    const long n = (long)B * wihi, total = n * C;
    int rc;
    if (training) {
        const int slices = (int)((n + SLICE - 1) / SLICE);
        float *ws = nullptr;
        if ((rc = conv_scratch((size_t)C * slices * sizeof(float4), &ws, st)) != TAGI_OK) return rc;
        float4 *part = reinterpret_cast<float4 *>(ws);
        if (wihi % 4 == 0 && aligned16(mu_a) && aligned16(var_a))
            bn2d_stats_partial_kernel<4><<<dim3(slices, C), BLOCK, 0, st>>>(mu_a, var_a, C, wihi, n, part);
        else
            bn2d_stats_partial_kernel<1><<<dim3(slices, C), BLOCK, 0, st>>>(mu_a, var_a, C, wihi, n, part);
        if ((rc = launched("bn2d_stats_partial_kernel launch")) != TAGI_OK) return rc;
        bn2d_stats_final_kernel<<<(C + 127) / 128, 128, 0, st>>>(part, slices, n, momentum, mu_batch, var_batch, mu_ra,
                                                                 var_ra, C);
        if ((rc = launched("bn2d_stats_final_kernel launch")) != TAGI_OK) return rc;
    }
    const float *mean = training ? mu_batch : mu_ra, *var = training ? var_batch : var_ra;
    if (wihi % 4 == 0 && aligned16(mu_a) && aligned16(var_a) && aligned16(mu_z) && aligned16(var_z))
        bn2d_apply_kernel<4><<<(unsigned)((total / 4 + BLOCK - 1) / BLOCK), BLOCK, 0, st>>>(
            mu_w, var_w, mu_b, var_b, mu_a, var_a, mean, var, eps, C, wihi, total, mu_z, var_z);
    else
        bn2d_apply_kernel<1><<<(unsigned)((total + BLOCK - 1) / BLOCK), BLOCK, 0, st>>>(
            mu_w, var_w, mu_b, var_b, mu_a, var_a, mean, var, eps, C, wihi, total, mu_z, var_z);
    return launched("bn2d_apply_kernel launch");
}

int bn2d_bwd(int B, int C, int wihi, int state_update, float eps, const float *mu_w, const float *var_w,
             const float *var_b, const float *mu_a, const float *jcb, const float *mu_batch, const float *var_batch,
             const float *dmu_o, const float *dvar_o, float *dmu, float *dvar, float *dmu_w, float *dvar_w, float *dmu_b,
             float *dvar_b, cudaStream_t st) {
    const long n = (long)B * wihi;
    const int slices = (int)((n + SLICE - 1) / SLICE);
    float *ws = nullptr;
    int rc;
    if ((rc = conv_scratch((size_t)C * slices * sizeof(float4), &ws, st)) != TAGI_OK) return rc;
    float4 *part = reinterpret_cast<float4 *>(ws);
    const bool vec = wihi % 4 == 0 && aligned16(mu_a) && aligned16(dmu_o) && aligned16(dvar_o) && (!jcb || aligned16(jcb)) &&
                     (!state_update || (aligned16(dmu) && aligned16(dvar)));
    if (vec)
        bn2d_bwd_kernel<4><<<dim3(slices, C), BLOCK, 0, st>>>(mu_w, var_w, mu_a, jcb, mu_batch, var_batch, dmu_o, dvar_o, eps,
                                                              C, wihi, n, state_update, dmu, dvar, part);
    else
        bn2d_bwd_kernel<1><<<dim3(slices, C), BLOCK, 0, st>>>(mu_w, var_w, mu_a, jcb, mu_batch, var_batch, dmu_o, dvar_o, eps,
                                                              C, wihi, n, state_update, dmu, dvar, part);
    if ((rc = launched("bn2d_bwd_kernel launch")) != TAGI_OK) return rc;
    bn2d_bwd_final_kernel<<<(C + 127) / 128, 128, 0, st>>>(part, slices, var_b, C, dmu_w, dvar_w, dmu_b, dvar_b);
    return launched("bn2d_bwd_final_kernel launch");
}

static PoolGeom pool_geom(const tagi_conv2d_geom &g) {
    PoolGeom p;
    p.C = g.fi, p.hi = g.hi, p.wi = g.wi, p.ho = g.ho, p.wo = g.wo, p.k = g.k, p.stride = g.stride;
    p.off = g.pad_type == 1 ? g.pad : 0;
    p.overlap = !(g.k == g.stride || g.k == g.wi);  // src/pooling_layer.cpp:188-191
    return p;
}

int avgpool2d_fwd(const tagi_conv2d_geom &g, const float *mu_a, const float *var_a, float *mu_z, float *var_z,
                  cudaStream_t st) {
    const long total = (long)g.B * g.fi * g.ho * g.wo;
    avgpool2d_fwd_kernel<<<(unsigned)((total + BLOCK - 1) / BLOCK), BLOCK, 0, st>>>(mu_a, var_a, pool_geom(g), total, mu_z,
                                                                                     var_z);
    return launched("avgpool2d_fwd_kernel launch");
}

int avgpool2d_bwd(const tagi_conv2d_geom &g, const float *jcb, const float *dmu_o, const float *dvar_o, float *dmu,
                  float *dvar, cudaStream_t st) {
    const long total = (long)g.B * g.fi * g.hi * g.wi;
    if (g.wi % 4 == 0 && aligned16(dmu) && aligned16(dvar) && (!jcb || aligned16(jcb)))
        avgpool2d_bwd_kernel<4><<<(unsigned)((total / 4 + BLOCK - 1) / BLOCK), BLOCK, 0, st>>>(
            jcb, dmu_o, dvar_o, pool_geom(g), (unsigned)(total / 4), dmu, dvar);
    else
        avgpool2d_bwd_kernel<1><<<(unsigned)((total + BLOCK - 1) / BLOCK), BLOCK, 0, st>>>(jcb, dmu_o, dvar_o, pool_geom(g),
                                                                                            (unsigned)total, dmu, dvar);
    return launched("avgpool2d_bwd_kernel launch");
}

int add_shortcut(size_t n, const float *mu_s, const float *var_s, const float *jcb, float *mu_a, float *var_a,
                 cudaStream_t st) {
    if (n == 0) return TAGI_OK;
    if (n % 4 == 0 && aligned16(mu_s) && aligned16(var_s) && aligned16(mu_a) && aligned16(var_a) && (!jcb || aligned16(jcb)))
        add_shortcut_vec4_kernel<<<(unsigned)((n / 4 + BLOCK - 1) / BLOCK), BLOCK, 0, st>>>(
            reinterpret_cast<const float4 *>(mu_s), reinterpret_cast<const float4 *>(var_s),
            reinterpret_cast<const float4 *>(jcb), n / 4, reinterpret_cast<float4 *>(mu_a), reinterpret_cast<float4 *>(var_a));
    else
        add_shortcut_kernel<<<(unsigned)((n + BLOCK - 1) / BLOCK), BLOCK, 0, st>>>(mu_s, var_s, jcb, n, mu_a, var_a);
    return launched("add_shortcut_kernel launch");
}

}  // namespace tagi

using namespace tagi;

#define TAGI_PTR(p) TAGI_REQUIRE((p) != nullptr && aligned4(p), #p " is null or not 4-byte aligned")

static int check_pool_geom(const tagi_conv2d_geom *g) {
    TAGI_REQUIRE(g != nullptr, "null geometry");
    TAGI_REQUIRE(g->B > 0 && g->fi > 0 && g->fi == g->fo, "B and the channel count (fi == fo) must be positive");
    TAGI_REQUIRE(g->k > 0 && g->stride > 0, "kernel and stride must be positive");
    int wo = 0, ho = 0;
    int rc = tagi_conv2d_out_size(g->k, g->stride, g->wi, g->hi, g->pad, g->pad_type, &wo, &ho);
    if (rc != TAGI_OK) return rc;
    TAGI_REQUIRE(wo == g->wo && ho == g->ho, "ho / wo do not match the kernel, stride and padding");
    TAGI_REQUIRE((long)g->B * g->fi * g->hi * g->wi < (1L << 31), "tensor extent exceeds 2^31 elements");
    return TAGI_OK;
}

extern "C" {

int tagi_bn2d_fwd(int B, int C, int wihi, int has_bias, int training, float eps, float momentum, const float *mu_w,
                  const float *var_w, const float *mu_b, const float *var_b, const float *mu_a, const float *var_a,
                  float *mu_ra, float *var_ra, float *mu_batch, float *var_batch, float *mu_z, float *var_z,
                  void *stream) {
    TAGI_REQUIRE(B > 0 && C > 0 && wihi > 0, "B, C and H*W must be positive");
    TAGI_REQUIRE((long)B * C * wihi < (1L << 31), "tensor extent exceeds 2^31 elements");
    TAGI_PTR(mu_w);
    TAGI_PTR(var_w);
    TAGI_PTR(mu_a);
    TAGI_PTR(var_a);
    TAGI_PTR(mu_ra);
    TAGI_PTR(var_ra);
    TAGI_PTR(mu_z);
    TAGI_PTR(var_z);
    if (has_bias) {
        TAGI_PTR(mu_b);
        TAGI_PTR(var_b);
    } else {
        mu_b = var_b = nullptr;
    }
    if (training) {
        TAGI_PTR(mu_batch);
        TAGI_PTR(var_batch);
    }
    return bn2d_fwd(B, C, wihi, training, eps, momentum, mu_w, var_w, mu_b, var_b, mu_a, var_a, mu_ra, var_ra, mu_batch,
                    var_batch, mu_z, var_z, static_cast<cudaStream_t>(stream));
}

int tagi_bn2d_bwd(int B, int C, int wihi, int has_bias, int state_update, float eps, const float *mu_w,
                  const float *var_w, const float *var_b, const float *mu_a, const float *jcb, const float *mu_batch,
                  const float *var_batch, const float *dmu_o, const float *dvar_o, float *dmu, float *dvar, float *dmu_w,
                  float *dvar_w, float *dmu_b, float *dvar_b, void *stream) {
    TAGI_REQUIRE(B > 0 && C > 0 && wihi > 0, "B, C and H*W must be positive");
    TAGI_REQUIRE((long)B * C * wihi < (1L << 31), "tensor extent exceeds 2^31 elements");
    TAGI_PTR(mu_w);
    TAGI_PTR(var_w);
    TAGI_PTR(mu_a);
    TAGI_PTR(mu_batch);
    TAGI_PTR(var_batch);
    TAGI_PTR(dmu_o);
    TAGI_PTR(dvar_o);
    TAGI_PTR(dmu_w);
    TAGI_PTR(dvar_w);
    if (state_update) {
        TAGI_PTR(dmu);
        TAGI_PTR(dvar);
    }
    if (has_bias) {
        TAGI_PTR(var_b);
        TAGI_PTR(dmu_b);
        TAGI_PTR(dvar_b);
    } else {
        var_b = nullptr;
    }
    return bn2d_bwd(B, C, wihi, state_update, eps, mu_w, var_w, var_b, mu_a, jcb, mu_batch, var_batch, dmu_o, dvar_o, dmu,
                    dvar, dmu_w, dvar_w, dmu_b, dvar_b, static_cast<cudaStream_t>(stream));
}

int tagi_avgpool2d_fwd(const tagi_conv2d_geom *g, const float *mu_a, const float *var_a, float *mu_z, float *var_z,
                       void *stream) {
    int rc = check_pool_geom(g);
    if (rc != TAGI_OK) return rc;
    TAGI_PTR(mu_a);
    TAGI_PTR(var_a);
    TAGI_PTR(mu_z);
    TAGI_PTR(var_z);
    return avgpool2d_fwd(*g, mu_a, var_a, mu_z, var_z, static_cast<cudaStream_t>(stream));
}

int tagi_avgpool2d_bwd_state(const tagi_conv2d_geom *g, const float *jcb, const float *dmu_o, const float *dvar_o,
                             float *dmu, float *dvar, void *stream) {
    int rc = check_pool_geom(g);
    if (rc != TAGI_OK) return rc;
    TAGI_PTR(dmu_o);
    TAGI_PTR(dvar_o);
    TAGI_PTR(dmu);
    TAGI_PTR(dvar);
    return avgpool2d_bwd(*g, jcb, dmu_o, dvar_o, dmu, dvar, static_cast<cudaStream_t>(stream));
}

int tagi_add_shortcut(const float *mu_s, const float *var_s, const float *jcb, size_t n, float *mu_a, float *var_a,
                      void *stream) {
    TAGI_PTR(mu_s);
    TAGI_PTR(var_s);
    TAGI_PTR(mu_a);
    TAGI_PTR(var_a);
    return add_shortcut(n, mu_s, var_s, jcb, mu_a, var_a, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
