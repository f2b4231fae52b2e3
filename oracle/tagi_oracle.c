/* CPU restatement of the reference's TAGI Linear / Conv2d arithmetic; see
 * tagi_oracle.h. TEST INFRASTRUCTURE ONLY. Built by `make -C oracle port` with
 * -ffp-contract=off so that, like the reference's baseline x86-64 build, no
 * multiply-add is fused. */
#include "tagi_oracle.h"

#include <math.h>

static int tagi_oracle_conv_offset(const tagi_oracle_conv_geom *g) { return g->pad_type == 1 ? g->pad : 0; }

int tagi_oracle_conv_out_size(int k, int stride, int wi, int hi, int pad, int pad_type, int *wo, int *ho) {
    int nw, nh;
    if (pad_type == 1) {
        nw = wi - k + 2 * pad;
        nh = hi - k + 2 * pad;
    } else if (pad_type == 2) {
        nw = wi - k + pad;
        nh = hi - k + pad;
    } else {
        nw = wi - k;
        nh = hi - k;
    }
    if (stride <= 0 || nw < 0 || nh < 0 || nw % stride || nh % stride) return -1;
    *wo = nw / stride + 1;
    *ho = nh / stride + 1;
    return 0;
}

#define ACC float
#define SUFFIX _f32
#include "tagi_oracle_body.inc"
#undef ACC
#undef SUFFIX

#define ACC double
#define SUFFIX _f64
#include "tagi_oracle_body.inc"
#undef ACC
#undef SUFFIX

void tagi_oracle_relu(size_t n, const float *mu_z, const float *var_z, float *mu_a, float *var_a, float *jcb) {
    for (size_t i = 0; i < n; i++) {
        float t = mu_z[i] > 0.0f ? mu_z[i] : 0.0f;
        mu_a[i] = t;
        if (t == 0.0f) {
            jcb[i] = 0.0f;
            var_a[i] = 0.0f;
        } else {
            jcb[i] = 1.0f;
            var_a[i] = var_z[i];
        }
    }
}

void tagi_oracle_mixture_relu(size_t n, const float *mu_z, const float *var_z, float *mu_a, float *var_a, float *jcb) {
    const float SQRT_2PI = 2.5066282746310002f;
    for (size_t i = 0; i < n; i++) {
        float m = mu_z[i];
        float sd = powf(var_z[i], 0.5f);
        float alpha = m / sd;
        float pdf = (1.0f / SQRT_2PI) * expf(-0.5f * alpha * alpha);
        float cdf = 0.5f * erfcf(-alpha * 0.7071067811865475f);
        float t = m * cdf + sd * pdf;
        mu_a[i] = fmaxf(0.000001f, t);
        var_a[i] = fmaxf(0.000001f, -t * t + 2 * t * m - m * sd * pdf + (var_z[i] - m * m) * cdf);
        jcb[i] = cdf;
    }
}

void tagi_oracle_output_delta(size_t n, const float *mu_a, const float *var_a, const float *jcb, const float *obs,
                              const float *var_obs, float *dmu, float *dvar) {
    for (size_t i = 0; i < n; i++) {
        float t = jcb[i] / (var_a[i] + var_obs[i]);
        if (isinf(t) || isnan(t) || isnan(obs[i])) {
            dmu[i] = 0.0f;
            dvar[i] = 0.0f;
        } else {
            dmu[i] = t * (obs[i] - mu_a[i]);
            dvar[i] = -t * jcb[i];
        }
    }
}

void tagi_oracle_output_delta_selected(int B, int n_out, int n_enc, const float *mu_a, const float *var_a,
                                       const float *jcb, const float *obs, const float *var_obs,
                                       const int *selected_idx, float *dmu, float *dvar) {
    for (long i = 0; i < (long)B * n_out; i++) dmu[i] = dvar[i] = 0.0f;
    for (long c = 0; c < (long)B * n_enc; c++) {
        long idx = selected_idx[c] + (c / n_enc) * n_out - 1;
        float t = jcb[idx] / (var_a[idx] + var_obs[c]);
        if (isinf(t) || isnan(t)) {
            dmu[idx] = 0.0f;
            dvar[idx] = 0.0f;
        } else {
            dmu[idx] = t * (obs[c] - mu_a[idx]);
            dvar[idx] = -t * jcb[idx];
        }
    }
}

int tagi_oracle_param_update(int batch_size, size_t n, float *mu, float *var, const float *dmu, const float *dvar) {
    /* cap factor: 0.1 for batch 1, 2 below 256, 3 from 256 on (src/base_layer.cpp:164-187) */
    float cap = batch_size == 1 ? 0.1f : (batch_size < 256 ? 2.0f : 3.0f);
    int neg = 0;
    for (size_t i = 0; i < n; i++) {
        float sm = (float)((dmu[i] > 0) - (dmu[i] < 0));
        float sv = (float)((dvar[i] > 0) - (dvar[i] < 0));
        float bar = powf(var[i], 0.5f) / cap;
        mu[i] += sm * fminf(fabsf(dmu[i]), bar);
        var[i] += sv * fminf(fabsf(dvar[i]), bar);
        if (var[i] <= 0.0f) {
            var[i] = 1e-5f;
            neg++;
        }
    }
    return neg;
}

/* ------------------------------------------------------------------ BatchNorm2d, AvgPool2d, residual add */
void tagi_oracle_bn2d_stats(int B, int C, int wihi, const float *mu_a, const float *var_a, float *mean, float *var) {
    int n = wihi * B;
#pragma omp parallel for schedule(static)
    for (int c = 0; c < C; c++) {
        float sm = 0.0f, sv = 0.0f;
        for (int i = 0; i < n; i++) {
            long idx = (long)(i / wihi) * wihi * C + i % wihi + (long)c * wihi;
            sm += mu_a[idx];
            sv += var_a[idx];
        }
        float m = sm / n;
        float s = 0.0f;
        for (int i = 0; i < n; i++) {
            long idx = (long)(i / wihi) * wihi * C + i % wihi + (long)c * wihi;
            s += (mu_a[idx] - m) * (mu_a[idx] - m);
        }
        mean[c] = m;
        var[c] = (s + sv) / (n - 1);
    }
}

void tagi_oracle_bn2d_running(int C, float momentum, const float *mean, const float *var, float *mu_ra, float *var_ra) {
    for (int c = 0; c < C; c++) {
        mu_ra[c] = mu_ra[c] * momentum + mean[c] * (1 - momentum);
        var_ra[c] = var_ra[c] * momentum + var[c] * (1 - momentum);
    }
}

void tagi_oracle_bn2d_fwd(int B, int C, int wihi, int has_bias, float eps, const float *mu_w, const float *var_w,
                          const float *mu_b, const float *var_b, const float *mu_a, const float *var_a,
                          const float *mean, const float *var, float *mu_z, float *var_z) {
#pragma omp parallel for schedule(static)
    for (int row = 0; row < B * C; row++) {
        int c = row % C;
        float inv = 1.0f / sqrtf(var[c] + eps);
        float m = mean[c], w = mu_w[c];
        for (int col = 0; col < wihi; col++) {
            long idx = col + (long)row * wihi;
            float t = mu_a[idx] - m;
            mu_z[idx] = inv * t * w;
            var_z[idx] = inv * inv * (var_a[idx] * (w * w + var_w[c]) + var_w[c] * t * t);
            if (has_bias) {
                mu_z[idx] += mu_b[c];
                var_z[idx] += var_b[c];
            }
        }
    }
}

void tagi_oracle_bn2d_bwd_state(int B, int C, int wihi, float eps, const float *mu_w, const float *jcb, const float *var,
                                const float *dmu_o, const float *dvar_o, float *dmu, float *dvar) {
#pragma omp parallel for schedule(static)
    for (int row = 0; row < B * C; row++) {
        int c = row % C;
        float inv = 1.0f / sqrtf(var[c] + eps);
        for (int col = 0; col < wihi; col++) {
            long idx = col + (long)row * wihi;
            float t = inv * mu_w[c] * jcb[idx];
            dmu[idx] = t * dmu_o[idx];
            dvar[idx] = t * dvar_o[idx] * t;
        }
    }
}

void tagi_oracle_bn2d_bwd_param(int B, int C, int wihi, int has_bias, float eps, const float *var_w, const float *var_b,
                                const float *mu_a, const float *mean, const float *var, const float *dmu_o,
                                const float *dvar_o, float *dmu_w, float *dvar_w, float *dmu_b, float *dvar_b) {
    int n = wihi * B;
#pragma omp parallel for schedule(static)
    for (int c = 0; c < C; c++) {
        float inv = 1.0f / sqrtf(var[c] + eps);
        float sm = 0.0f, sv = 0.0f, bm = 0.0f, bv = 0.0f;
        for (int i = 0; i < n; i++) {
            long idx = (long)(i / wihi) * wihi * C + i % wihi + (long)c * wihi;
            float t = inv * (mu_a[idx] - mean[c]) * var_w[c];
            sm += t * dmu_o[idx];
            sv += t * dvar_o[idx] * t;
            if (has_bias) {
                float tb = var_b[c];
                bm += tb * dmu_o[idx];
                bv += tb * dvar_o[idx] * tb;
            }
        }
        dmu_w[c] = sm;
        dvar_w[c] = sv;
        if (has_bias) {
            dmu_b[c] = bm;
            dvar_b[c] = bv;
        }
    }
}

void tagi_oracle_avgpool2d_fwd(const tagi_oracle_conv_geom *g, const float *mu_a, const float *var_a, float *mu_z,
                               float *var_z) {
    const int off = tagi_oracle_conv_offset(g), k2 = g->k * g->k, woho = g->wo * g->ho, wihi = g->wi * g->hi;
    const long planes = (long)g->B * g->fi;
#pragma omp parallel for schedule(static)
    for (long pl = 0; pl < planes; pl++)
        for (int p = 0; p < woho; p++) {
            int oy = p / g->wo, ox = p % g->wo;
            float sm = 0.0f, sv = 0.0f;
            for (int t = 0; t < k2; t++) { /* taps in row-major order, as the index table lists them */
                int y = oy * g->stride - off + t / g->k, x = ox * g->stride - off + t % g->k;
                if (y < 0 || y >= g->hi || x < 0 || x >= g->wi) continue;
                sm += mu_a[pl * wihi + (long)y * g->wi + x];
                sv += var_a[pl * wihi + (long)y * g->wi + x];
            }
            mu_z[pl * woho + p] = sm / k2;
            var_z[pl * woho + p] = sv / (k2 * k2);
        }
}

void tagi_oracle_avgpool2d_bwd_state(const tagi_oracle_conv_geom *g, const float *jcb, const float *dmu_o,
                                     const float *dvar_o, float *dmu, float *dvar) {
    const int off = tagi_oracle_conv_offset(g), k2 = g->k * g->k, woho = g->wo * g->ho, wihi = g->wi * g->hi;
    const long planes = (long)g->B * g->fi;
    const int overlap = !(g->k == g->stride || g->k == g->wi);
#pragma omp parallel for schedule(static)
    for (long pl = 0; pl < planes; pl++)
        for (int q = 0; q < wihi; q++) {
            int y = q / g->wi, x = q % g->wi;
            long i = pl * wihi + q;
            if (!overlap) { /* one cell per pixel, no sum (src/pooling_layer.cpp:355-375) */
                /* k == stride: the cell of the pixel; k == wi (global pooling): the only cell */
                int oy = g->k == g->stride ? y / g->k : 0, ox = g->k == g->stride ? x / g->k : 0;
                float dm = 0.0f, dv = 0.0f;
                if (oy < g->ho && ox < g->wo) {
                    dm = dmu_o[pl * woho + (long)oy * g->wo + ox];
                    dv = dvar_o[pl * woho + (long)oy * g->wo + ox];
                }
                dmu[i] = dm * jcb[i] / k2;
                dvar[i] = dv * jcb[i] * jcb[i] / (k2 * k2);
                continue;
            }
            float sm = 0.0f, sv = 0.0f;
            /* cells that contain the pixel, in the order of the reference's table: descending tap index */
            for (int t = k2 - 1; t >= 0; t--) {
                int ty = y + off - t / g->k, tx = x + off - t % g->k;
                if (ty < 0 || tx < 0 || ty % g->stride || tx % g->stride) continue;
                int oy = ty / g->stride, ox = tx / g->stride;
                if (oy >= g->ho || ox >= g->wo) continue;
                sm += dmu_o[pl * woho + (long)oy * g->wo + ox];
                sv += dvar_o[pl * woho + (long)oy * g->wo + ox];
            }
            dmu[i] = sm * jcb[i] / k2;
            dvar[i] = sv * jcb[i] * jcb[i] / (k2 * k2);
        }
}

void tagi_oracle_add_shortcut(size_t n, const float *mu_s, const float *var_s, const float *jcb, float *mu_a,
                              float *var_a) {
    for (size_t i = 0; i < n; i++) {
        if (jcb) {
            mu_a[i] += mu_s[i] * jcb[i];
            var_a[i] += var_s[i] * jcb[i] * jcb[i];
        } else {
            mu_a[i] += mu_s[i];
            var_a[i] += var_s[i];
        }
    }
}
