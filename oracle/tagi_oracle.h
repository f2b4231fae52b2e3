/* CPU restatement of the reference's TAGI Linear / Conv2d arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY: the parity tests, the smoke check and the CPU leg
 * of the benchmark call this; the product library never does.
 *
 * Pinning: the reference ships no golden vectors or op-level tests for Linear
 * or Conv2d, so this restatement is pinned by the reference's own CPU classes
 * executed in the build container (oracle/_ref/libtagi_ref.so, built by
 * oracle/Makefile from the reference's sources) and by the fixtures under
 * tests/golden/ that were generated from those classes.
 *
 * Layouts (row-major, flat): activations / deltas [B][features]; Linear weights
 * [N][K]; conv activations [B][C][H][W], conv weights [fo][fi][k][k], conv
 * outputs [B][fo][ho*wo].
 */
#ifndef TAGI_ORACLE_H
#define TAGI_ORACLE_H
#include <stddef.h>
#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
    int B, fi, hi, wi, fo, ho, wo, k, stride, pad, pad_type, has_bias;
} tagi_oracle_conv_geom;

/* Output extent, src/conv2d_layer.cpp:581-628: pad_type 1 -> (w - k + 2p)/s + 1,
 * pad_type 2 -> (w - k + p)/s + 1, else (w - k)/s + 1. Returns -1 (the reference
 * raises) when the numerator is not divisible by the stride. */
int tagi_oracle_conv_out_size(int k, int stride, int wi, int hi, int pad, int pad_type, int *wo, int *ho);

#define TAGI_ORACLE_DECL(ACC, S)                                                                                  \
    void tagi_oracle_linear_fwd##S(int B, int K, int N, int has_bias, const float *mu_w, const float *var_w,      \
                                   const float *mu_b, const float *var_b, const float *mu_a, const float *var_a,  \
                                   ACC *mu_z, ACC *var_z);                                                        \
    void tagi_oracle_linear_bwd_state##S(int B, int K, int N, const float *mu_w, const float *jcb,                \
                                         const float *dmu_z, const float *dvar_z, ACC *dmu_a, ACC *dvar_a);       \
    void tagi_oracle_linear_bwd_param##S(int B, int K, int N, int has_bias, const float *var_w,                   \
                                         const float *var_b, const float *mu_a, const float *dmu_z,               \
                                         const float *dvar_z, ACC *dmu_w, ACC *dvar_w, ACC *dmu_b, ACC *dvar_b);  \
    void tagi_oracle_conv2d_fwd##S(const tagi_oracle_conv_geom *g, const float *mu_w, const float *var_w,         \
                                   const float *mu_b, const float *var_b, const float *mu_a, const float *var_a,  \
                                   ACC *mu_z, ACC *var_z);                                                        \
    void tagi_oracle_conv2d_bwd_state##S(const tagi_oracle_conv_geom *g, const float *mu_w, const float *jcb,     \
                                         const float *dmu_z, const float *dvar_z, ACC *dmu_a, ACC *dvar_a);       \
    void tagi_oracle_conv2d_bwd_param##S(const tagi_oracle_conv_geom *g, const float *var_w, const float *var_b,  \
                                         const float *mu_a, const float *dmu_z, const float *dvar_z, ACC *dmu_w,  \
                                         ACC *dvar_w, ACC *dmu_b, ACC *dvar_b);
TAGI_ORACLE_DECL(float, _f32)
TAGI_ORACLE_DECL(double, _f64)

/* Neighbours of the path, fp32 elementwise, needed to run whole training steps. */
/* ReLU moments, src/activation.cpp:7-29. */
void tagi_oracle_relu(size_t n, const float *mu_z, const float *var_z, float *mu_a, float *var_a, float *jcb);
/* MixtureReLU moments (rectified Gaussian), src/activation.cpp:152-178: alpha = mu_z / sqrt(var_z),
 * mu_a = max(1e-6, mu_z * Phi(alpha) + sqrt(var_z) * phi(alpha)), var_a likewise floored, jcb = Phi(alpha). */
void tagi_oracle_mixture_relu(size_t n, const float *mu_z, const float *var_z, float *mu_a, float *var_a, float *jcb);
/* Output innovation, src/base_output_updater.cpp:8-29: all n entries. */
void tagi_oracle_output_delta(size_t n, const float *mu_a, const float *var_a, const float *jcb, const float *obs,
                              const float *var_obs, float *dmu, float *dvar);
/* Index-selected innovation (hierarchical softmax), src/base_output_updater.cpp:67-93: dmu/dvar (B*n_out entries)
 * are zeroed first (src/base_output_updater.cpp:281,300), then n_sel = B*n_enc entries are written; selected_idx
 * is one-based within a sample. */
void tagi_oracle_output_delta_selected(int B, int n_out, int n_enc, const float *mu_a, const float *var_a,
                                       const float *jcb, const float *obs, const float *var_obs,
                                       const int *selected_idx, float *dmu, float *dvar);
/* Capped parameter update, src/base_layer.cpp:116-187; returns how many variances were reset to 1e-5. */
int tagi_oracle_param_update(int batch_size, size_t n, float *mu, float *var, const float *dmu, const float *dvar);


/* ---- layers around Conv2d in the CNN / ResNet configurations (fp32, activations [B][C][H*W]) ---- */
/* BatchNorm2d batch statistics in training, src/batchnorm_layer.cpp:127-168: mean[c] = sum mu_a / n,
 * var[c] = (sum (mu_a - mean)^2 + sum var_a) / (n - 1), n = B * wihi, sums over (b, pixel) in that order. */
void tagi_oracle_bn2d_stats(int B, int C, int wihi, const float *mu_a, const float *var_a, float *mean, float *var);
/* Running averages, src/batchnorm_layer.cpp:15-26: ra = ra * momentum + batch * (1 - momentum). */
void tagi_oracle_bn2d_running(int C, float momentum, const float *mean, const float *var, float *mu_ra, float *var_ra);
/* Normalisation with the given statistics, src/batchnorm_layer.cpp:170-206. */
void tagi_oracle_bn2d_fwd(int B, int C, int wihi, int has_bias, float eps, const float *mu_w, const float *var_w,
                          const float *mu_b, const float *var_b, const float *mu_a, const float *var_a,
                          const float *mean, const float *var, float *mu_z, float *var_z);
/* State deltas, src/batchnorm_layer.cpp:233-255. */
void tagi_oracle_bn2d_bwd_state(int B, int C, int wihi, float eps, const float *mu_w, const float *jcb, const float *var,
                                const float *dmu_o, const float *dvar_o, float *dmu, float *dvar);
/* Parameter deltas, src/batchnorm_layer.cpp:307-357 followed by delta_param_sum (src/common.cpp:360-376). */
void tagi_oracle_bn2d_bwd_param(int B, int C, int wihi, int has_bias, float eps, const float *var_w, const float *var_b,
                                const float *mu_a, const float *mean, const float *var, const float *dmu_o,
                                const float *dvar_o, float *dmu_w, float *dvar_w, float *dmu_b, float *dvar_b);
/* AvgPool2d, src/pooling_layer.cpp:207-283 (forward) and :285-353 (state deltas), with the receptive field of
 * src/indices.cpp (same rule as Conv2d: input pixel (oy*s - off + ky, ox*s - off + kx), off = pad for padding type 1,
 * 0 with bottom/right padding for type 2); taps in the padding contribute nothing, the divisor stays k*k.
 * g->fi = g->fo = channels, has_bias unused. */
void tagi_oracle_avgpool2d_fwd(const tagi_oracle_conv_geom *g, const float *mu_a, const float *var_a, float *mu_z,
                               float *var_z);
void tagi_oracle_avgpool2d_bwd_state(const tagi_oracle_conv_geom *g, const float *jcb, const float *dmu_o,
                                     const float *dvar_o, float *dmu, float *dvar);
/* Residual connection, src/resnet_block.cpp:8-31: a += s (states, or deltas of a projection shortcut) and
 * a += s * j, va += vs * j * j (identity shortcut, j = Jacobian of the block input). jcb may be NULL (= 1). */
void tagi_oracle_add_shortcut(size_t n, const float *mu_s, const float *var_s, const float *jcb, float *mu_a,
                              float *var_a);

#ifdef __cplusplus
}
#endif
#endif
