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
