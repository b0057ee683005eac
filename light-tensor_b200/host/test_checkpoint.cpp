// Writes a quantized checkpoint from CPU modules filled by a fixed recipe, reloads it into fresh modules and compares.
// Needs no GPU.  The file it leaves behind (argv[1]) is also read by the Python loader in tests/test_checkpoint.py, which
// knows the recipe: byte i of tensor number t = (7*i + t) mod 251, int32 element i = 1000*i - 7*t, zero points
// 10+m / 20+m / 30+m and weight scale 0.5/(m+1) for module m.
#include <stdio.h>
#include <string.h>

#include <vector>

#include "lten_q.h"

using namespace lten;

static void fill(std::vector<Module *> &mods)
{
    int t = 0;
    for (size_t m = 0; m < mods.size(); m++) {
        for (Tensor *w : mods[m]->get_all_weights()) {
            const uint64_t n = w->get_numels();
            if (w->get_data_type() == UINT8) {
                uint8_t *p = (uint8_t *)w->get_data_ptr();
                for (uint64_t i = 0; i < n; i++) p[i] = (uint8_t)((7 * i + t) % 251);
            } else {
                int32_t *p = (int32_t *)w->get_data_ptr();
                for (uint64_t i = 0; i < n; i++) p[i] = (int32_t)(1000 * i) - 7 * t;
            }
            t++;
        }
        QuantizationParams qw{0.5f / (float)(m + 1), (uint8_t)(20 + m)};
        mods[m]->set_qparams_in(QuantizationParams{0.25f, (uint8_t)(10 + m)});
        mods[m]->set_qparams_out(QuantizationParams{2.f, (uint8_t)(30 + m)});
        mods[m]->set_qparams_params(&qw, 1);
    }
}

static std::vector<Module *> build()
{
    std::vector<Module *> mods = {new Conv2d_q(2, 5, true, 3, 3, 1, 1), new FullyConnected_q(20, 7, true),
                                  new FullyConnected_q(7, 3, false)};
    for (Module *m : mods) m->init();
    return mods;
}

int main(int argc, char **argv)
{
    if (argc < 2) return 2;
    std::vector<Module *> a = build(), b = build();
    fill(a);
    if (save_checkpoint(a, argv[1]) != 0) {
        printf("FAIL: save\n");
        return 1;
    }
    if (load_checkpoint(b, argv[1]) != 0) {
        printf("FAIL: load\n");
        return 1;
    }
    int bad = 0;
    for (size_t m = 0; m < a.size(); m++) {
        std::vector<Tensor *> ta = a[m]->get_all_weights(), tb = b[m]->get_all_weights();
        for (size_t i = 0; i < ta.size(); i++) {
            const size_t bytes = ta[i]->get_numels() * (ta[i]->get_data_type() == UINT8 ? 1 : 4);
            bad += memcmp(ta[i]->get_data_ptr(), tb[i]->get_data_ptr(), bytes) != 0;
        }
        QuantizationParams qa[3], qb[3];
        a[m]->get_qparams(qa);
        b[m]->get_qparams(qb);
        for (int i = 0; i < 3; i++) bad += qa[i].scale != qb[i].scale || qa[i].zero_point != qb[i].zero_point;
    }
    std::vector<Module *> fewer(b.begin(), b.begin() + 2);
    bad += load_checkpoint(fewer, argv[1]) == 0;  // module count mismatch must be refused
    for (Module *m : a) delete m;
    for (Module *m : b) delete m;
    if (bad) {
        printf("FAIL: %d mismatches\n", bad);
        return 1;
    }
    printf("PASS\n");
    return 0;
}
