// Compile-time tables of the layer-1 tensor product: which (output l, harmonic l1, feature l2)
// paths exist for a given highest feature degree, and where each path's blocks live in the
// flattened arrays. The enumeration rule is the one behind the reference's Phi1_l / Phi1_l1 /
// Phi1_l2 model arrays (symmetrix/source/symmetrix/extract_mace_data.py:323-342): feature degree
// outermost, then harmonic degree, then output degree, natural parity, outputs up to l = 3,
// stably sorted by output degree. The model loader maps the file's own path order onto this one.
#pragma once

namespace smx {

constexpr int kLmaxSH = 3;    // spherical-harmonic degree of the edge attributes (fixed, as in the reference)
constexpr int kNumLm = 16;    // (kLmaxSH + 1)^2
constexpr int kMaxPaths = 24;

struct TPTable {
    int P = 0;                    // number of paths
    int l[kMaxPaths] = {};        // output degree
    int l1[kMaxPaths] = {};       // harmonic degree
    int l2[kMaxPaths] = {};       // feature degree
    int e[kMaxPaths] = {};        // rank of the path among paths with the same output degree
    int n_e[kLmaxSH + 1] = {};    // paths per output degree
    int lme_off[kLmaxSH + 1] = {};// first output slot of each output degree: sum_{l'<l} (2l'+1) n_e(l')
    int zoff[kMaxPaths] = {};     // first entry of the path's (2l+1) x (2l2+1) coupling block
    int toff[kMaxPaths] = {};     // first entry of the path's (2l1+1) x (2l2+1) block (reference index lelm1lm2)
    int NZ = 0;                   // sum_p (2l+1)(2l2+1)
    int T = 0;                    // sum_p (2l1+1)(2l2+1)   (reference num_lelm1lm2)
    int Q = 0;                    // sum_p (2l+1)           (reference num_lme)
    int nLM = 0;                  // (L_max + 1)^2

    // output slot of (path p, m index 0..2l): lme_off[l] + m * n_e[l] + e[p]
    constexpr int lme(int p, int m) const { return lme_off[l[p]] + m * n_e[l[p]] + e[p]; }
};

constexpr TPTable make_tp_table(int L_max) {
    TPTable t{};
    t.nLM = (L_max + 1) * (L_max + 1);
    // enumerate in generation order, then stable-sort by l (insertion by output degree)
    int gl[kMaxPaths] = {}, gl1[kMaxPaths] = {}, gl2[kMaxPaths] = {};
    int n = 0;
    for (int l2 = 0; l2 <= L_max; ++l2)
        for (int l1 = 0; l1 <= kLmaxSH; ++l1) {
            const int lo = l1 > l2 ? l1 - l2 : l2 - l1;
            const int hi = (l1 + l2 < kLmaxSH) ? l1 + l2 : kLmaxSH;
            for (int l = lo; l <= hi; ++l)
                if ((l1 + l2 + l) % 2 == 0) {
                    gl[n] = l; gl1[n] = l1; gl2[n] = l2; ++n;
                }
        }
    int p = 0;
    for (int l = 0; l <= kLmaxSH; ++l)
        for (int i = 0; i < n; ++i)
            if (gl[i] == l) {
                t.l[p] = l; t.l1[p] = gl1[i]; t.l2[p] = gl2[i];
                t.e[p] = t.n_e[l];
                t.n_e[l] += 1;
                ++p;
            }
    t.P = p;
    int off = 0;
    for (int l = 0; l <= kLmaxSH; ++l) {
        t.lme_off[l] = off;
        off += (2 * l + 1) * t.n_e[l];
    }
    t.Q = off;
    for (int q = 0; q < t.P; ++q) {
        t.zoff[q] = t.NZ;
        t.toff[q] = t.T;
        t.NZ += (2 * t.l[q] + 1) * (2 * t.l2[q] + 1);
        t.T += (2 * t.l1[q] + 1) * (2 * t.l2[q] + 1);
    }
    return t;
}

}  // namespace smx
