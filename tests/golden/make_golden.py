"""Makes tests/golden/reference_vectors.json from the reference's own C code.

What of prabanta-dev/janas compiles alone on a CPU is compiled here (gcc) and run
on small inputs: its sampler (src/llm/sample.c with src/llm/jmath.c), its
math functions for RoPE angles and the activated gate (janas_powf,
janas_sincosf in src/llm/jmath.c; janas_silu_mul_det in src/llm/vmath.h), and
its attention (src/llm/attention.c: janas_attn_run with float scores) over keys
and values that its eight-bit cache holds exactly (a byte times a scale per
position and KV head), in blocks of 50 tokens, with and without a window, and
its RMSNorm (rms_norm, an inline function of src/llm/model_impl.h).  The
whole model cannot be run this way (it takes quantized weights only), so the
plain implementation in tests/plain_qwen3.py rests on the formulas for the rest.

    python tests/golden/make_golden.py /path/to/prabanta-dev/janas

The inputs are made by a 64-bit LCG that tests/test_plain.py repeats, so the
JSON holds only the outputs.
"""
import json
import os
import subprocess
import sys
import tempfile

DRIVER = r'''
#include <stdio.h>
#include <stdint.h>
#include <stdlib.h>
#include "sample.h"
#include "jmath.h"
#include "vmath.h"

static uint64_t lcg_state;
static double lcg(void) { /* uniform in [0, 1) */
    lcg_state = lcg_state * 6364136223846793005ull + 1442695040888963407ull;
    return (double)(lcg_state >> 11) * (1.0 / 9007199254740992.0);
}

int main(void)
{
    const int V = 300, ROWS = 12;
    static float rows[12][300];
    lcg_state = 12345;
    for (int r = 0; r < ROWS; r++)
        for (int i = 0; i < V; i++)
            rows[r][i] = (float)((lcg() - 0.5) * 8.0);
    /* exact ties: equal logits at the top and around a top_k cut */
    rows[3][17] = rows[3][5] = 6.0f;
    rows[4][100] = rows[4][101] = rows[4][102] = 3.5f;
    struct { float t; int k; float p, mp; uint64_t seed; } S[] = {
        {0.0f, 0, 0.0f, 0.0f, 1}, {0.8f, 20, 0.8f, 0.0f, 1}, {0.7f, 0, 0.0f, 0.0f, 7},
        {1.0f, 5, 0.0f, 0.0f, 42}, {1.5f, 0, 0.9f, 0.05f, 3}, {0.3f, 50, 1.0f, 0.2f, 99},
        {2.0f, 3, 0.5f, 0.0f, 18446744073709551615ull}};
    printf("{\"sampler\": [");
    for (unsigned s = 0; s < sizeof S / sizeof *S; s++) {
        struct janas_sampler *sm = janas_sampler_create(V);
        struct janas_sample_params p = {S[s].t, S[s].k, S[s].p, S[s].mp, 0, 0, -1};
        janas_sampler_set(sm, &p, S[s].seed);
        printf("%s[", s ? ", " : "");
        for (int rep = 0; rep < 3; rep++)
            for (int r = 0; r < ROWS; r++)
                printf("%s%d", rep + r ? ", " : "", janas_sampler_pick(sm, rows[r], NULL));
        printf("]");
        janas_sampler_destroy(sm);
    }
    printf("],\n \"rope\": [");
    float bases[] = {10000.0f, 1000000.0f, 50000.0f};
    int nrot[] = {16, 32, 128};
    int pos[] = {0, 1, 7, 63, 64, 1000, 8191, 40000};
    int first = 1;
    for (int b = 0; b < 3; b++)
        for (int pi = 0; pi < 8; pi++)
            for (int i = 0; i < nrot[b] / 2; i += (nrot[b] / 8)) {
                float theta = (float)pos[pi] * janas_powf(bases[b], -2.0f * (float)i / (float)nrot[b]);
                float sn, cs;
                janas_sincosf(theta, &sn, &cs);
                printf("%s[%d, %d, %d, %.9g, %.9g]", first ? "" : ", ", b, pos[pi], i, cs, sn);
                first = 0;
            }
    printf("],\n \"silu_mul\": [");
    lcg_state = 777;
    for (int i = 0; i < 40; i++) {
        float g = (float)((lcg() - 0.5) * 24.0), u = (float)((lcg() - 0.5) * 4.0);
        printf("%s%.9g", i ? ", " : "", janas_silu_mul_det(g, u));
    }
    printf("]}\n");
    return 0;
}
'''

ATTENTION_DRIVER = r'''
#include <stdio.h>
#include <stdint.h>
#include <stdlib.h>
#include "attention.h"
#include "common/pool.h"

static uint64_t lcg_state;
static double lcg(void) {
    lcg_state = lcg_state * 6364136223846793005ull + 1442695040888963407ull;
    return (double)(lcg_state >> 11) * (1.0 / 9007199254740992.0);
}

int main(void)
{
    /* heads, KV heads, head size, tokens, window, seed; the rows that are printed */
    struct { int nh, nkv, hd, n, window; uint64_t seed; int rows[6]; } C[] = {
        {4, 2, 16, 70, 0, 11, {0, 1, 49, 50, 64, 69}},
        {5, 1, 48, 150, 37, 12, {0, 36, 37, 63, 100, 149}},
        {6, 3, 128, 300, 150, 13, {0, 149, 150, 255, 256, 299}}};
    struct janas_pool *pool = janas_pool_create(1, NULL);
    printf("{\"attention\": [");
    for (unsigned c = 0; c < sizeof C / sizeof *C; c++) {
        int nh = C[c].nh, nkv = C[c].nkv, hd = C[c].hd, n = C[c].n;
        uint32_t n_ctx = 512;
        float *q = malloc(sizeof(float) * n * nh * hd), *out = malloc(sizeof(float) * n * nh * hd);
        int8_t *k = calloc((size_t)nkv * n_ctx * hd, 1), *v = calloc((size_t)nkv * n_ctx * hd, 1);
        float *ks = calloc((size_t)nkv * n_ctx, sizeof(float));
        float *vs = calloc((size_t)nkv * n_ctx, sizeof(float));
        lcg_state = C[c].seed;
        for (int i = 0; i < n * nh * hd; i++)
            q[i] = (float)((lcg() - 0.5) * 4.0);
        for (int h = 0; h < nkv; h++)
            for (int t = 0; t < n; t++) {
                ks[h * n_ctx + t] = (float)(0.004 + 0.008 * lcg());
                vs[h * n_ctx + t] = (float)(0.004 + 0.008 * lcg());
                for (int d = 0; d < hd; d++) {
                    k[((size_t)h * n_ctx + t) * hd + d] = (int8_t)((int)(lcg() * 255.0) - 127);
                    v[((size_t)h * n_ctx + t) * hd + d] = (int8_t)((int)(lcg() * 255.0) - 127);
                }
            }
        struct janas_attn *a = janas_attn_create(nh, nkv, hd, n_ctx, 1, JANAS_ATTN_FLOAT);
        if (!a || janas_attn_scores_mode(a) != JANAS_ATTN_FLOAT)
            return 1;
        if (C[c].window)
            janas_attn_set_window(a, C[c].window);
        for (int p0 = 0; p0 < n; p0 += 50) {      /* at most 64 tokens a call */
            int cnt = n - p0 < 50 ? n - p0 : 50;
            janas_attn_run(a, pool, q + (size_t)p0 * nh * hd, k, ks, v, vs, cnt, p0,
                           out + (size_t)p0 * nh * hd);
        }
        printf("%s{\"nh\": %d, \"nkv\": %d, \"hd\": %d, \"n\": %d, \"window\": %d, "
               "\"seed\": %llu, \"rows\": {", c ? ", " : "", nh, nkv, hd, n, C[c].window,
               (unsigned long long)C[c].seed);
        int step = hd / 16;                        /* sixteen values of every head */
        for (int r = 0; r < 6; r++) {
            printf("%s\"%d\": [", r ? ", " : "", C[c].rows[r]);
            for (int h = 0; h < nh; h++)
                for (int d = 0; d < hd; d += step)
                    printf("%s%.9g", h + d ? ", " : "",
                           out[((size_t)C[c].rows[r] * nh + h) * hd + d]);
            printf("]");
        }
        printf("}}");
        janas_attn_destroy(a);
        free(q); free(out); free(k); free(v); free(ks); free(vs);
    }
    printf("]}\n");
    janas_pool_destroy(pool);
    return 0;
}
'''

NORM_DRIVER = r'''
#include <stdio.h>
#include <stdint.h>
#include <stdlib.h>
#include "model_impl.h"

static uint64_t lcg_state;
static double lcg(void) {
    lcg_state = lcg_state * 6364136223846793005ull + 1442695040888963407ull;
    return (double)(lcg_state >> 11) * (1.0 / 9007199254740992.0);
}

int main(void)
{
    struct { int n; float eps; uint64_t seed; } C[] = {
        {16, 1e-6f, 21}, {96, 1e-5f, 22}, {104, 3e-6f, 23}, {2560, 1e-6f, 24}};
    printf("{\"rms_norm\": [");
    for (unsigned c = 0; c < sizeof C / sizeof *C; c++) {
        int n = C[c].n;
        float *x = malloc(sizeof(float) * n), *w = malloc(sizeof(float) * n);
        float *out = malloc(sizeof(float) * n);
        lcg_state = C[c].seed;
        for (int i = 0; i < n; i++) {
            x[i] = (float)((lcg() - 0.5) * 8.0);
            w[i] = (float)(1.0 + (lcg() - 0.5) * 0.4);
        }
        rms_norm(out, x, w, (uint32_t)n, C[c].eps);
        int step = n > 128 ? n / 16 : 1;
        printf("%s{\"n\": %d, \"eps\": %.9g, \"seed\": %llu, \"step\": %d, \"out\": [",
               c ? ", " : "", n, C[c].eps, (unsigned long long)C[c].seed, step);
        for (int i = 0; i < n; i += step)
            printf("%s%.9g", i ? ", " : "", out[i]);
        printf("]}");
        free(x); free(w); free(out);
    }
    printf("]}\n");
    return 0;
}
'''


def main():
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    ref = sys.argv[1]
    here = os.path.dirname(os.path.abspath(__file__))
    with tempfile.TemporaryDirectory() as tmp:
        drv = os.path.join(tmp, "driver.c")
        with open(drv, "w") as f:
            f.write(DRIVER)
        exe = os.path.join(tmp, "driver")
        subprocess.run(["gcc", "-O2", "-ffp-contract=off", "-I", os.path.join(ref, "src/llm"),
                        "-I", os.path.join(ref, "src"), drv,
                        os.path.join(ref, "src/llm/sample.c"),
                        os.path.join(ref, "src/llm/jmath.c"), "-lm", "-o", exe], check=True)
        out = subprocess.run([exe], check=True, capture_output=True, text=True).stdout
        drv = os.path.join(tmp, "attention_driver.c")
        with open(drv, "w") as f:
            f.write(ATTENTION_DRIVER)
        exe = os.path.join(tmp, "attention_driver")
        llm, common = os.path.join(ref, "src/llm"), os.path.join(ref, "src/common")
        subprocess.run(["gcc", "-O2", "-ffp-contract=off", "-I", llm, "-I", os.path.join(ref, "src"),
                        drv] + [os.path.join(llm, f) for f in
                                ("attention.c", "jmath.c", "quant.c", "quant_q6k.c", "tuner.c")]
                       + [os.path.join(common, f) for f in
                          ("pool.c", "sysinfo.c", "paths.c", "cpu_features.c")]
                       + ["-lm", "-lpthread", "-o", exe], check=True)
        # the reference keeps tuning notes below HOME: give it the scratch folder
        att = subprocess.run([exe], check=True, capture_output=True, text=True,
                             env=dict(os.environ, HOME=tmp, JANAS_ATTN="float")).stdout
        # rms_norm is an inline function of the model's own header
        drv = os.path.join(tmp, "norm_driver.c")
        with open(drv, "w") as f:
            f.write(NORM_DRIVER)
        exe = os.path.join(tmp, "norm_driver")
        subprocess.run(["gcc", "-O2", "-ffp-contract=off", "-I", llm, "-I", os.path.join(ref, "src"),
                        "-I", os.path.join(ref, "include"), drv, os.path.join(llm, "jmath.c"),
                        "-lm", "-o", exe], check=True)
        norm = subprocess.run([exe], check=True, capture_output=True, text=True).stdout
    data = json.loads(out)
    data.update(json.loads(att))
    data.update(json.loads(norm))
    with open(os.path.join(here, "reference_vectors.json"), "w") as f:
        json.dump(data, f)
        f.write("\n")
    print("wrote", os.path.join(here, "reference_vectors.json"),
          {k: len(v) for k, v in data.items()})


if __name__ == "__main__":
    main()
