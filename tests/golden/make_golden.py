"""Makes tests/golden/reference_vectors.json from the reference's own C code.

What of prabanta-dev/janas compiles alone on a CPU is compiled here (gcc) and run
on small inputs: its sampler (src/llm/sample.c with src/llm/jmath.c) and its
math functions for RoPE angles and the activated gate (janas_powf,
janas_sincosf in src/llm/jmath.c; janas_silu_mul_det in src/llm/vmath.h).  The
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
    data = json.loads(out)
    with open(os.path.join(here, "reference_vectors.json"), "w") as f:
        json.dump(data, f)
        f.write("\n")
    print("wrote", os.path.join(here, "reference_vectors.json"),
          {k: len(v) for k, v in data.items()})


if __name__ == "__main__":
    main()
