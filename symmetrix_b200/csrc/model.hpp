// Host-side model: reads a symmetrix JSON model file and prepares the tables the kernels use.
// Replaces MACE::load_from_json (libsymmetrix/source/mace.cpp:905-1030; device twin
// mace_kokkos.cpp:1544-1887). Everything is kept in double here; the evaluator casts to its
// arithmetic type when uploading.
#pragma once

#include <algorithm>
#include <array>
#include <cmath>
#include <fstream>
#include <limits>
#include <map>
#include <sstream>
#include <string>
#include <vector>

#include "json_min.hpp"
#include "tp_tables.hpp"
#include "generated/cg_canon.hpp"
#include "generated/poly_canon.hpp"

namespace smx {

struct ModelError : std::runtime_error {
    using std::runtime_error::runtime_error;
};
struct UnsupportedError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

// A sparse polynomial of degree <= 3 in the 16 variables A[i, :, k], shared by all channels and
// element types (which only change the coefficients), compiled to a flat operation stream for the
// nested Horner form
//   P = sum_q1 A[q1] (c1 + sum_{q2} A[q2] (c2 + sum_{q3} c3 A[q3])).
// One 32-bit word per operation: kind | variable << 3 | (coefficient row + 1) << 8, where the row
// is the monomial's position in the model's monomial list (0: no such monomial, coefficient zero).
// A flat stream lets the kernels fetch the coefficients of later operations while executing the
// current one. Takes the place of the product DAG the reference builds per (element, LM, channel)
// (libsymmetrix/source/multivariate_polynomial.cpp:10-101).
enum PolyOp : int { kPolyLeaf = 0, kPolyPairBegin = 1, kPolyPairEnd = 2, kPolyHeadBegin = 3, kPolyHeadEnd = 4, kPolyNop = 5 };
constexpr int kPolyPrefetch = 8;     // operations fetched ahead; streams are padded with this many no-ops

struct PolyProgram {
    std::vector<int> words;
    int num_monomials = 0;
    int num_leaves = 0, num_pairs = 0;
    std::vector<int> alias;      // alias[mu]: the monomial whose coefficient row the program reads for monomial mu (mu itself
                                 // unless the list repeats a monomial: then the first occurrence, whose row must hold the sum)
};

inline int poly_word(int kind, int q, int mu) { return kind | (q << 3) | ((mu + 1) << 8); }

inline PolyProgram compile_polynomial(const std::vector<std::vector<int>>& monomials, int num_vars) {
    struct Pair { int mu = -1; std::vector<std::pair<int, int>> leaves; };
    struct Head { int mu = -1; std::map<int, Pair> pairs; };
    std::map<int, Head> heads;
    std::vector<int> alias(monomials.size());
    for (size_t mu = 0; mu < monomials.size(); ++mu) {
        alias[mu] = static_cast<int>(mu);
        std::vector<int> m = monomials[mu];
        std::sort(m.begin(), m.end());
        if (m.empty() || m.size() > 3) throw UnsupportedError("symmetric contraction: monomial degree must be 1..3");
        for (int q : m)
            if (q < 0 || q >= num_vars) throw ModelError("symmetric contraction: variable index out of range");
        Head& h = heads[m[0]];
        if (m.size() == 1) { if (h.mu < 0) h.mu = static_cast<int>(mu); else alias[mu] = h.mu; continue; }
        Pair& p = h.pairs[m[1]];
        if (m.size() == 2) { if (p.mu < 0) p.mu = static_cast<int>(mu); else alias[mu] = p.mu; continue; }
        bool dup = false;
        for (auto& lf : p.leaves)
            if (lf.first == m[2]) { dup = true; alias[mu] = lf.second; }
        if (!dup) p.leaves.emplace_back(m[2], static_cast<int>(mu));
    }
    PolyProgram prog;
    prog.alias = alias;
    prog.num_monomials = static_cast<int>(monomials.size());
    for (auto& [q1, h] : heads) {
        prog.words.push_back(poly_word(kPolyHeadBegin, q1, h.mu));
        for (auto& [q2, p] : h.pairs) {
            prog.words.push_back(poly_word(kPolyPairBegin, q2, p.mu));
            prog.num_pairs += 1;
            for (auto& lf : p.leaves) {
                prog.words.push_back(poly_word(kPolyLeaf, lf.first, lf.second));
                prog.num_leaves += 1;
            }
            prog.words.push_back(poly_word(kPolyPairEnd, q2, -1));
        }
        prog.words.push_back(poly_word(kPolyHeadEnd, q1, -1));
    }
    while (prog.words.size() % kPolyPrefetch) prog.words.push_back(poly_word(kPolyNop, 0, -1));
    for (int i = 0; i < kPolyPrefetch; ++i) prog.words.push_back(poly_word(kPolyNop, 0, -1));
    return prog;
}

struct HostModel {
    // basic information (mace.hpp:18-25)
    int num_elements = 0, K = 0, l_max = 0, L_max = 0, num_lm = 0, num_LM = 0;
    double r_cut = 0.0;
    std::vector<int> atomic_numbers;
    std::vector<double> atomic_energies;
    bool has_zbl = false;
    // ZBL pair repulsion (zbl.hpp:43-56): exponent / prefactor of the screening length, 4 screening coefficients,
    // covalent radii indexed by atomic number, envelope order
    double zbl_a_exp = 0.0, zbl_a_prefactor = 0.0;
    std::vector<double> zbl_c, zbl_covalent_radii;
    int zbl_p = 0;
    // density normalisation of the two interaction layers (mace.cpp:273-346, 681-757): scalar cubic splines per
    // unordered element pair, coefficients [pair][bin][4] (cubic_spline.cpp:55-71)
    bool A0_scaled = false, A1_scaled = false;
    double A0_spline_h = 0.0, A1_spline_h = 0.0;
    int A0_spline_bins = 0, A1_spline_bins = 0;
    std::vector<double> A0_spline_coef, A1_spline_coef;

    // radial splines: coefficient tables [pair][bin][function][4] (cubic_spline_set.cpp:5-25)
    double spline_h = 0.0;
    int num_bins = 0;                // G - 1
    int num_pairs = 0;               // E (E + 1) / 2 unordered pairs
    int F0 = 0, F1 = 0;              // functions per pair: (l_max+1) K and P K
    std::vector<double> coef0, coef1;

    std::vector<double> H0_w;        // [E][K]
    std::vector<double> A0_w;        // [E][l_max+1][K][K]
    std::vector<double> H1_w;        // [L_max+1][K][K]
    std::vector<double> A1_w;        // concatenated per l: [n_e(l) K][K], path blocks in canonical order
    std::array<long, kLmaxSH + 2> A1_w_off{};
    std::vector<double> H2_w_H1;     // [E][K][K]
    std::vector<double> H2_w_M1;     // [K][K]
    std::vector<double> ro1;         // [K]
    std::vector<double> ro2_w1;      // [16][K]
    std::vector<double> ro2_w2;      // [16]
    double ro2_scale = 1.0;

    // tensor product: canonical path table; the file's Clebsch-Gordan COO must equal the canonical non-zeros
    // (generated/cg_canon.hpp) up to one scale per path, which is folded into that path's radial functions
    TPTable tp{};
    std::vector<int> path_file_to_canon;   // index by the file's path number
    std::vector<int> lme_file_to_canon;    // output slot permutation (identity for canonical files)
    std::vector<double> path_scale;        // per canonical path: file coupling / canonical coupling
    // Un-splined radial network of interaction block 1 (optional extra keys "x_radial_*" of a model file; what the
    // reference's exporter tabulates into the splines, extract_mace_data.py:144-172):
    //   basis_n(r) = sqrt(2 / r_cut) sin(n pi r / r_cut) / r * cutoff_p(r / r_cut) * pair_scale[pair][n],  n = 1..num_bessel
    //   x <- silu_scale * silu(x W_i) for the hidden layers,  R = x W_last
    // `w_last` is in canonical path order with the per-path coupling scale folded in, like the spline tables.
    struct RadialMlp {
        bool present = false;
        int num_bessel = 0, poly_p = 0, hidden = 0, num_hidden_layers = 0;
        double silu_scale = 1.0;
        std::vector<double> w_first;      // [num_bessel][hidden]
        std::vector<double> w_hidden;     // [num_hidden_layers - 1][hidden][hidden]
        std::vector<double> w_last;       // [hidden][P K]
        std::vector<double> pair_scale;   // [pairs][num_bessel]
        // Low-rank form of the radial tables (optional keys x_radial_basis_*_1): the last hidden layer tabulated on the
        // spline grid, as cubic coefficients [pair][bin][hidden][4]. Spline construction and the last layer are both
        // linear, so (these) x w_last reproduces the radial spline tables to rounding.
        std::vector<double> basis_coef;
    } rmlp1;

    // symmetric contractions: programs per LM (M0) and one for M1; coefficients [element][monomial][K]
    std::vector<PolyProgram> prog0;
    std::vector<int> mono_off0;            // first monomial row of each LM in coef_M0
    int num_mono0 = 0;
    std::vector<double> coef_M0;
    PolyProgram prog1;
    int num_mono1 = 0;
    std::vector<double> coef_M1;
    // the same coefficients re-ordered to the canonical monomial lists (generated/poly_canon.hpp) used by the
    // straight-line kernels; `poly_canonical` is false if the file has monomials outside those lists
    bool poly_canonical = true;
    int num_canon0 = 0, num_canon1 = 0;
    std::vector<double> coef_M0_canon, coef_M1_canon;

    // Optional middle interaction block (file key "num_interactions": 3; an extension of the reference's two-block
    // format, whose exporter stops at two blocks, extract_mace_data.py:70-71). Same tensor-product tables as the last
    // block, a contraction that keeps every (L, M) like M0, a per-L linear plus a per-element, per-L residual of H1.
    int num_interactions = 2;
    std::vector<double> coefm;             // radial splines, as coef1
    std::vector<double> Am_w;              // as A1_w
    std::array<long, kLmaxSH + 2> Am_w_off{};
    std::vector<PolyProgram> progm;        // as prog0
    std::vector<int> mono_offm;
    int num_monom = 0, num_canonm = 0;
    std::vector<double> coef_Mm, coef_Mm_canon;
    std::vector<double> Hm_w;              // [L_max+1][K][K]
    std::vector<double> Hm_res;            // [E][L_max+1][K][K]
    std::vector<double> ro_m;              // [K]
};

namespace detail {
// slot of each of the file's monomials of output component `lm` in the canonical list, or -1
inline std::vector<int> canonical_slots(const std::vector<std::vector<int>>& monomials, int lm) {
    std::vector<int> out(monomials.size(), -1);
    for (size_t mu = 0; mu < monomials.size(); ++mu) {
        std::vector<int> m = monomials[mu];
        std::sort(m.begin(), m.end());
        m.resize(3, -1);
        for (int s = 0; s < kCanonPolyCount[lm]; ++s) {
            const CanonMonomial& c = kCanonMonomials[kCanonPolyOffset[lm] + s];
            if (c.q[0] == m[0] && c.q[1] == m[1] && c.q[2] == m[2]) { out[mu] = s; break; }
        }
    }
    return out;
}
}  // namespace detail

namespace detail {

inline std::vector<std::vector<int>> int_lists(const JsonValue& v) {
    std::vector<std::vector<int>> out;
    if (v.type == JsonValue::NumArray && v.nums.empty()) return out;
    if (v.type != JsonValue::Array) throw ModelError("model file: expected a list of index lists");
    for (const auto& row : v.arr) out.push_back(row.flat_int());
    return out;
}

// Spline coefficients of one pair table: values/derivs [F][G] -> c[bin][F][4], formulas of
// CubicSplineSet::CubicSplineSet (cubic_spline_set.cpp:13-24).
inline void spline_coefficients(const JsonValue& values, const JsonValue& derivs, double h, int F, int G,
                                const std::vector<int>& fn_map, double* c) {
    if (static_cast<int>(values.size()) != F || static_cast<int>(derivs.size()) != F)
        throw ModelError("model file: radial spline table has the wrong number of functions");
    for (int f = 0; f < F; ++f) {
        const auto& v = values.arr.empty() ? values : values.arr[f];
        const auto& d = derivs.arr.empty() ? derivs : derivs.arr[f];
        if (v.type != JsonValue::NumArray || d.type != JsonValue::NumArray ||
            static_cast<int>(v.nums.size()) != G || static_cast<int>(d.nums.size()) != G)
            throw ModelError("model file: radial spline table has ragged rows");
        const int fo = fn_map.empty() ? f : fn_map[f];
        for (int i = 0; i < G - 1; ++i) {
            double* o = c + (static_cast<size_t>(i) * F + fo) * 4;
            const double v0 = v.nums[i], v1 = v.nums[i + 1], d0 = d.nums[i], d1 = d.nums[i + 1];
            o[0] = v0;
            o[1] = d0;
            o[2] = (-3 * v0 - 2 * h * d0 + 3 * v1 - h * d1) / (h * h);
            o[3] = (2 * v0 + h * d0 - 2 * v1 + h * d1) / (h * h * h);
        }
    }
}

}  // namespace detail

inline HostModel load_model_file(const std::string& filename) {
    std::ifstream f(filename, std::ios::binary);
    if (!f) throw ModelError("cannot open model file '" + filename + "'");
    std::string text((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
    JsonValue file = JsonParser(text.data(), text.data() + text.size()).parse();
    text.clear();
    text.shrink_to_fit();
    if (file.type != JsonValue::Object) throw JsonError("[json] model file is not a JSON object");

    HostModel m;
    m.num_elements = file.at("num_elements").as_int();
    m.K = file.at("num_channels").as_int();
    m.r_cut = file.at("r_cut").as_double();
    m.l_max = file.at("l_max").as_int();
    m.L_max = file.at("L_max").as_int();
    m.num_lm = (m.l_max + 1) * (m.l_max + 1);
    m.num_LM = (m.L_max + 1) * (m.L_max + 1);
    m.atomic_numbers = file.at("atomic_numbers").flat_int();
    m.atomic_energies = file.at("atomic_energies").flat();
    m.has_zbl = file.at("has_zbl").as_bool();
    const int E = m.num_elements, K = m.K;
    if (static_cast<int>(m.atomic_numbers.size()) != E || static_cast<int>(m.atomic_energies.size()) != E)
        throw ModelError("model file: atomic_numbers / atomic_energies do not match num_elements");
    if (m.l_max != kLmaxSH) throw UnsupportedError("only l_max == 3 is supported (as in the reference exporter)");
    if (m.L_max < 0 || m.L_max > 3) throw UnsupportedError("hidden features up to L_max == 3 are supported");
    if (K < 1 || K > 1024) throw UnsupportedError("num_channels must be in 1..1024");
    if (m.has_zbl) {
        m.zbl_a_exp = file.at("zbl_a_exp").as_double();
        m.zbl_a_prefactor = file.at("zbl_a_prefactor").as_double();
        m.zbl_c = file.at("zbl_c").flat();
        m.zbl_covalent_radii = file.at("zbl_covalent_radii").flat();
        m.zbl_p = file.at("zbl_p").as_int();
        if (m.zbl_c.size() != 4) throw ModelError("model file: zbl_c needs 4 coefficients");
        for (int z : m.atomic_numbers)
            if (z < 0 || z >= static_cast<int>(m.zbl_covalent_radii.size())) throw ModelError("model file: zbl_covalent_radii does not cover the model's elements");
    }
    auto load_scalar_splines = [&](const char* hkey, const char* vkey, const char* dkey, double& h, int& bins, std::vector<double>& coef) {
        h = file.at(hkey).as_double();
        const JsonValue& vals = file.at(vkey);
        const JsonValue& ders = file.at(dkey);
        const int pairs = E * (E + 1) / 2;
        if (vals.type != JsonValue::Array || static_cast<int>(vals.size()) != pairs || static_cast<int>(ders.size()) != pairs)
            throw ModelError(std::string("model file: ") + vkey + " must have one spline per unordered element pair");
        const int G = static_cast<int>(vals.arr[0].size());
        if (G < 2) throw ModelError("model file: density splines need at least two nodes");
        bins = G - 1;
        coef.assign(static_cast<size_t>(pairs) * bins * 4, 0.0);
        for (int pr = 0; pr < pairs; ++pr) {
            const auto& v = vals.arr[pr].nums;
            const auto& d = ders.arr[pr].nums;
            if (static_cast<int>(v.size()) != G || static_cast<int>(d.size()) != G) throw ModelError("model file: ragged density spline table");
            for (int i = 0; i < bins; ++i) {   // CubicSpline::generate_coefficients, cubic_spline.cpp:61-69
                double* o = coef.data() + (static_cast<size_t>(pr) * bins + i) * 4;
                o[0] = v[i];
                o[1] = d[i];
                o[2] = (-3 * o[0] - 2 * h * o[1] + 3 * v[i + 1] - h * d[i + 1]) / (h * h);
                o[3] = (2 * o[0] + h * o[1] - 2 * v[i + 1] + h * d[i + 1]) / (h * h * h);
            }
        }
    };
    m.A0_scaled = file.at("A0_scaled").as_bool();
    m.A1_scaled = file.at("A1_scaled").as_bool();
    if (m.A0_scaled) load_scalar_splines("A0_spline_h", "A0_spline_values", "A0_spline_derivs", m.A0_spline_h, m.A0_spline_bins, m.A0_spline_coef);
    if (m.A1_scaled) load_scalar_splines("A1_spline_h", "A1_spline_values", "A1_spline_derivs", m.A1_spline_h, m.A1_spline_bins, m.A1_spline_coef);

    // ---- tensor-product paths: map the file's order onto the canonical table
    m.tp = make_tp_table(m.L_max);
    const std::vector<int> pl = file.at("Phi1_l").flat_int(), pl1 = file.at("Phi1_l1").flat_int(),
                           pl2 = file.at("Phi1_l2").flat_int();
    const int P = static_cast<int>(pl.size());
    if (P != m.tp.P || pl1.size() != pl.size() || pl2.size() != pl.size())
        throw UnsupportedError("tensor-product path list differs from the standard l_max=3 enumeration");
    m.path_file_to_canon.assign(P, -1);
    std::vector<int> file_e(P, 0), file_ne(kLmaxSH + 1, 0);
    for (int p = 0; p < P; ++p) {
        if (p > 0 && pl[p] < pl[p - 1]) throw ModelError("Phi1_l must be sorted by non-decreasing l");
        if (pl[p] < 0 || pl[p] > kLmaxSH) throw ModelError("Phi1_l out of range");
        file_e[p] = file_ne[pl[p]]++;
        for (int c = 0; c < m.tp.P; ++c)
            if (m.tp.l[c] == pl[p] && m.tp.l1[c] == pl1[p] && m.tp.l2[c] == pl2[p]) m.path_file_to_canon[p] = c;
        if (m.path_file_to_canon[p] < 0) throw UnsupportedError("tensor-product path not in the standard enumeration");
    }
    {
        std::vector<int> seen(P, 0);
        for (int c : m.path_file_to_canon) seen[c] += 1;
        for (int s : seen) if (s != 1) throw UnsupportedError("duplicate tensor-product path");
    }
    // file lme / t decoders
    std::vector<int> file_lme_off(kLmaxSH + 2, 0), file_toff(P + 1, 0);
    for (int l = 0; l <= kLmaxSH; ++l) file_lme_off[l + 1] = file_lme_off[l] + (2 * l + 1) * file_ne[l];
    for (int p = 0; p < P; ++p) file_toff[p + 1] = file_toff[p] + (2 * pl1[p] + 1) * (2 * pl2[p] + 1);
    m.lme_file_to_canon.assign(m.tp.Q, -1);
    for (int p = 0; p < P; ++p) {
        const int l = pl[p], c = m.path_file_to_canon[p];
        for (int mm = 0; mm < 2 * l + 1; ++mm)
            m.lme_file_to_canon[file_lme_off[l] + mm * file_ne[l] + file_e[p]] = m.tp.lme(c, mm);
    }
    {   // compare the file's coupling entries with the canonical non-zeros, path by path
        const std::vector<int> cg_lme = file.at("Phi1_lme").flat_int(), cg_t = file.at("Phi1_lelm1lm2").flat_int();
        const std::vector<double> cg_c = file.at("Phi1_clebsch_gordan").flat();
        if (cg_lme.size() != cg_c.size() || cg_t.size() != cg_c.size())
            throw ModelError("model file: Clebsch-Gordan COO arrays differ in length");
        const CanonCG* canon = nullptr;
        int n_canon = 0;
        switch (m.L_max) {
            case 0: canon = CanonCGTable<0>::e; n_canon = CanonCGTable<0>::n; break;
            case 1: canon = CanonCGTable<1>::e; n_canon = CanonCGTable<1>::n; break;
            case 2: canon = CanonCGTable<2>::e; n_canon = CanonCGTable<2>::n; break;
            default: canon = CanonCGTable<3>::e; n_canon = CanonCGTable<3>::n; break;
        }
        std::vector<double> file_val(n_canon, 0.0);
        std::vector<int> hits(n_canon, 0);
        for (size_t n = 0; n < cg_c.size(); ++n) {
            const int t = cg_t[n], lme = cg_lme[n];
            if (t < 0 || t >= file_toff[P] || lme < 0 || lme >= m.tp.Q) throw ModelError("Clebsch-Gordan index out of range");
            int p = 0;
            while (t >= file_toff[p + 1]) ++p;
            const int l = pl[p], l1 = pl1[p], l2 = pl2[p];
            const int rem = t - file_toff[p];
            const int i1 = rem / (2 * l2 + 1), i2 = rem % (2 * l2 + 1);
            const int rel = lme - file_lme_off[l];   // the output slot must belong to the same path
            if (rel < 0 || rel >= (2 * l + 1) * file_ne[l] || rel % file_ne[l] != file_e[p])
                throw ModelError("Clebsch-Gordan entry couples a path to another path's output slot");
            const int mm = rel / file_ne[l];
            const int c = m.path_file_to_canon[p];
            int found = -1;
            for (int q = 0; q < n_canon; ++q)
                if (canon[q].p == c && canon[q].m == mm && canon[q].lm1 == l1 * l1 + i1 && canon[q].lm2 == l2 * l2 + i2) { found = q; break; }
            if (found < 0) {
                if (std::fabs(cg_c[n]) < 1e-10) continue;
                throw UnsupportedError("Clebsch-Gordan entry outside the real-harmonics coupling pattern of the evaluator");
            }
            file_val[found] += cg_c[n];
            hits[found] += 1;
        }
        m.path_scale.assign(m.tp.P, 0.0);
        for (int c = 0; c < m.tp.P; ++c) {
            double num = 0.0, den = 0.0;
            for (int q = 0; q < n_canon; ++q)
                if (canon[q].p == c) { num += file_val[q] * canon[q].c; den += canon[q].c * canon[q].c; }
            const double scale = num / den;    // least-squares scale of this path
            for (int q = 0; q < n_canon; ++q)
                if (canon[q].p == c && std::fabs(file_val[q] - scale * canon[q].c) > 1e-9 * std::max(1.0, std::fabs(scale)))
                    throw UnsupportedError("Clebsch-Gordan values of a path are not proportional to the evaluator's coupling table");
            m.path_scale[c] = scale;
        }
    }

    // ---- radial splines
    m.spline_h = file.at("radial_spline_h").as_double();
    m.num_pairs = E * (E + 1) / 2;
    m.F0 = (m.l_max + 1) * K;
    m.F1 = P * K;
    auto load_splines = [&](const char* vkey, const char* dkey, int F, const std::vector<int>& fn_map,
                            std::vector<double>& out) {
        const JsonValue& vals = file.at(vkey);
        const JsonValue& ders = file.at(dkey);
        if (static_cast<int>(vals.size()) != m.num_pairs || static_cast<int>(ders.size()) != m.num_pairs || vals.type != JsonValue::Array)
            throw ModelError(std::string("model file: ") + vkey + " must have one table per unordered element pair");
        const JsonValue& first = vals.arr[0];
        if (first.type != JsonValue::Array || first.arr.empty()) throw ModelError("model file: empty radial spline table");
        const int G = static_cast<int>(first.arr[0].size());
        if (G < 2) throw ModelError("model file: radial splines need at least two nodes");
        if (m.num_bins == 0) m.num_bins = G - 1;
        if (m.num_bins != G - 1) throw ModelError("model file: radial spline tables differ in length");
        out.assign(static_cast<size_t>(m.num_pairs) * (G - 1) * F * 4, 0.0);
        for (int pr = 0; pr < m.num_pairs; ++pr)
            detail::spline_coefficients(vals.arr[pr], ders.arr[pr], m.spline_h, F, G, fn_map,
                                        out.data() + static_cast<size_t>(pr) * (G - 1) * F * 4);
    };
    load_splines("radial_spline_values_0", "radial_spline_derivs_0", m.F0, {}, m.coef0);
    std::vector<int> fn_map(m.F1);
    for (int p = 0; p < P; ++p)
        for (int k = 0; k < K; ++k) fn_map[p * K + k] = m.path_file_to_canon[p] * K + k;
    load_splines("radial_spline_values_1", "radial_spline_derivs_1", m.F1, fn_map, m.coef1);
    auto fold_path_scale = [&](std::vector<double>& coef) {   // per-path coupling scale into the radial functions of that path
        const size_t rows = static_cast<size_t>(m.num_pairs) * m.num_bins;
        for (size_t row = 0; row < rows; ++row)
            for (int c = 0; c < m.tp.P; ++c) {
                const double sc = m.path_scale[c];
                if (sc == 1.0) continue;
                double* o = coef.data() + (row * m.F1 + static_cast<size_t>(c) * K) * 4;
                for (int q = 0; q < 4 * K; ++q) o[q] *= sc;
            }
    };
    fold_path_scale(m.coef1);
    if (const JsonValue* dims_v = file.find("x_radial_mlp_dims_1")) {
        HostModel::RadialMlp& r = m.rmlp1;
        const std::vector<int> dims = dims_v->flat_int();
        const JsonValue& ws = file.at("x_radial_mlp_weights_1");
        r.num_bessel = file.at("x_radial_num_bessel").as_int();
        r.poly_p = file.at("x_radial_poly_p").as_int();
        r.silu_scale = file.at("x_radial_silu_scale").as_double();
        // supported shape: num_bessel -> hidden -> ... -> hidden -> P K with at least one hidden layer of equal widths
        bool ok = dims.size() >= 3 && ws.size() + 1 == dims.size() && dims.front() == r.num_bessel && dims.back() == m.F1 &&
                  r.num_bessel >= 1 && r.num_bessel <= 16;
        for (size_t i = 2; ok && i + 1 < dims.size(); ++i) ok = dims[i] == dims[1];
        if (ok && (dims[1] < 1 || dims[1] > 64)) ok = false;
        if (ok) {
            r.hidden = dims[1];
            r.num_hidden_layers = static_cast<int>(dims.size()) - 2;
            r.w_first = ws.arr[0].flat();
            for (int i = 1; i < r.num_hidden_layers; ++i) {
                const std::vector<double> w = ws.arr[i].flat();
                if (w.size() != static_cast<size_t>(r.hidden) * r.hidden) ok = false;
                r.w_hidden.insert(r.w_hidden.end(), w.begin(), w.end());
            }
            const std::vector<double> last = ws.arr[ws.size() - 1].flat();
            r.pair_scale = file.at("x_radial_pair_scale_1").flat();
            if (r.w_first.size() != static_cast<size_t>(r.num_bessel) * r.hidden || last.size() != static_cast<size_t>(r.hidden) * m.F1 ||
                r.pair_scale.size() != static_cast<size_t>(m.num_pairs) * r.num_bessel) ok = false;
            if (ok) {
                r.w_last.assign(last.size(), 0.0);
                for (int j = 0; j < r.hidden; ++j)
                    for (int pf = 0; pf < P; ++pf) {
                        const int c = m.path_file_to_canon[pf];
                        for (int k = 0; k < K; ++k)
                            r.w_last[static_cast<size_t>(j) * m.F1 + c * K + k] = m.path_scale[c] * last[static_cast<size_t>(j) * m.F1 + pf * K + k];
                    }
            }
        }
        if (!ok) throw ModelError("model file: x_radial_* keys are inconsistent (expected num_bessel -> equal hidden layers -> num_paths * num_channels)");
        r.present = true;
        if (const JsonValue* bv = file.find("x_radial_basis_values_1")) {
            const JsonValue& bd = file.at("x_radial_basis_derivs_1");
            if (static_cast<int>(bv->size()) != m.num_pairs || static_cast<int>(bd.size()) != m.num_pairs)
                throw ModelError("model file: x_radial_basis_*_1 must have one table per unordered element pair");
            const int G = m.num_bins + 1;
            r.basis_coef.assign(static_cast<size_t>(m.num_pairs) * m.num_bins * r.hidden * 4, 0.0);
            for (int pr = 0; pr < m.num_pairs; ++pr)
                detail::spline_coefficients(bv->arr[pr], bd.arr[pr], m.spline_h, r.hidden, G, {},
                                            r.basis_coef.data() + static_cast<size_t>(pr) * m.num_bins * r.hidden * 4);
        }
    }
    if (const JsonValue* ni = file.find("num_interactions")) m.num_interactions = ni->as_int();
    if (m.num_interactions != 2 && m.num_interactions != 3) throw UnsupportedError("num_interactions must be 2 or 3");
    if (m.num_interactions == 3) {
        if (m.has_zbl || m.A0_scaled || m.A1_scaled)
            throw UnsupportedError("ZBL / density normalisation are not defined for models with three interaction blocks");
        load_splines("radial_spline_values_m", "radial_spline_derivs_m", m.F1, fn_map, m.coefm);
        fold_path_scale(m.coefm);
    }

    // ---- dense weights
    auto expect = [&](const std::vector<double>& v, size_t n, const char* key) {
        if (v.size() != n) throw ModelError(std::string("model file: ") + key + " has the wrong size");
    };
    m.H0_w = file.at("H0_weights").flat();  expect(m.H0_w, size_t(E) * K, "H0_weights");
    m.A0_w = file.at("A0_weights").flat();  expect(m.A0_w, size_t(E) * (m.l_max + 1) * K * K, "A0_weights");
    m.H1_w = file.at("H1_weights").flat();  expect(m.H1_w, size_t(m.L_max + 1) * K * K, "H1_weights");
    auto load_A_weights = [&](const char* key, std::vector<double>& out, std::array<long, kLmaxSH + 2>& offs) {
        const JsonValue& a1 = file.at(key);
        if (static_cast<int>(a1.size()) != m.l_max + 1) throw ModelError(std::string("model file: ") + key + " needs one matrix per l");
        long off = 0;
        for (int l = 0; l <= m.l_max; ++l) {
            std::vector<double> w = a1.arr.empty() ? std::vector<double>() : a1.arr[l].flat();
            const int ne = m.tp.n_e[l];
            expect(w, size_t(ne) * K * K, key);
            offs[l] = off;
            out.resize(off + long(ne) * K * K);
            // permute the e-blocks of rows from file order to canonical order
            for (int p = 0; p < P; ++p) {
                if (pl[p] != l) continue;
                const int ec = m.tp.e[m.path_file_to_canon[p]];
                std::copy(w.begin() + long(file_e[p]) * K * K, w.begin() + long(file_e[p] + 1) * K * K,
                          out.begin() + off + long(ec) * K * K);
            }
            off += long(ne) * K * K;
        }
        offs[m.l_max + 1] = off;
    };
    load_A_weights("A1_weights", m.A1_w, m.A1_w_off);
    if (m.num_interactions == 3) {
        load_A_weights("Am_weights", m.Am_w, m.Am_w_off);
        m.Hm_w = file.at("Hm_weights").flat();            expect(m.Hm_w, size_t(m.L_max + 1) * K * K, "Hm_weights");
        m.Hm_res = file.at("Hm_weights_for_H1").flat();   expect(m.Hm_res, size_t(E) * (m.L_max + 1) * K * K, "Hm_weights_for_H1");
        m.ro_m = file.at("readout_m_weights").flat();     expect(m.ro_m, K, "readout_m_weights");
    }
    m.H2_w_H1 = file.at("H2_weights_for_H1").flat();  expect(m.H2_w_H1, size_t(E) * K * K, "H2_weights_for_H1");
    m.H2_w_M1 = file.at("H2_weights_for_M1").flat();  expect(m.H2_w_M1, size_t(K) * K, "H2_weights_for_M1");
    m.ro1 = file.at("readout_1_weights").flat();      expect(m.ro1, K, "readout_1_weights");
    m.ro2_w1 = file.at("readout_2_weights_1").flat(); expect(m.ro2_w1, size_t(16) * K, "readout_2_weights_1");
    m.ro2_w2 = file.at("readout_2_weights_2").flat(); expect(m.ro2_w2, 16, "readout_2_weights_2");
    m.ro2_scale = file.at("readout_2_scale_factor").as_double();

    // ---- symmetric contractions
    auto load_full_contraction = [&](const char* mono_key, const char* weight_key, std::vector<PolyProgram>& prog,
                                     std::vector<int>& mono_off, int& num_mono, std::vector<double>& coef, int& num_canon,
                                     std::vector<double>& coef_canon) {
        const JsonValue& monos = file.at(mono_key);
        const JsonValue& weights = file.at(weight_key);
        mono_off.assign(m.num_LM + 1, 0);
        for (int lm = 0; lm < m.num_LM; ++lm) {
            auto lists = detail::int_lists(monos.at(std::to_string(lm)));
            prog.push_back(compile_polynomial(lists, m.num_lm));
            mono_off[lm + 1] = mono_off[lm] + static_cast<int>(lists.size());
        }
        num_mono = mono_off[m.num_LM];
        coef.assign(size_t(E) * num_mono * K, 0.0);
        // the straight-line contraction kernels exist for outputs up to L = 2 (9 components); beyond that the table-driven
        // kernels run the file's own monomial lists
        constexpr int kCanonOutputs = static_cast<int>(sizeof(kCanonPolyCount) / sizeof(kCanonPolyCount[0]));
        const bool have_canon = m.num_LM <= kCanonOutputs;
        if (!have_canon) m.poly_canonical = false;
        num_canon = have_canon ? kCanonPolyOffset[m.num_LM] : 0;
        coef_canon.assign(size_t(E) * num_canon * K, 0.0);
        std::vector<std::vector<int>> slots0;
        for (int lm = 0; lm < m.num_LM; ++lm) {
            auto lists = detail::int_lists(monos.at(std::to_string(lm)));
            slots0.push_back(have_canon ? detail::canonical_slots(lists, lm) : std::vector<int>(lists.size(), -1));
            for (int sl : slots0.back()) if (sl < 0) m.poly_canonical = false;
        }
        for (int a = 0; a < E; ++a) {
            const JsonValue& wa = weights.at(std::to_string(a));
            for (int lm = 0; lm < m.num_LM; ++lm) {
                const JsonValue& wl = wa.at(std::to_string(lm));
                const int nm = mono_off[lm + 1] - mono_off[lm];
                for (int k = 0; k < K; ++k) {
                    const JsonValue& wk = wl.at(std::to_string(k));
                    if (static_cast<int>(wk.size()) != nm) throw ModelError(std::string(weight_key) + " row length differs from " + mono_key);
                    for (int mu = 0; mu < nm; ++mu) {
                        // a monomial listed twice contributes the sum of its coefficients (as the reference's product DAG does)
                        coef[(size_t(a) * num_mono + mono_off[lm] + prog[prog.size() - m.num_LM + lm].alias[mu]) * K + k] += wk.nums[mu];
                        if (slots0[lm][mu] >= 0)
                            coef_canon[(size_t(a) * num_canon + kCanonPolyOffset[lm] + slots0[lm][mu]) * K + k] += wk.nums[mu];
                    }
                }
            }
        }
    };
    load_full_contraction("M0_monomials", "M0_weights", m.prog0, m.mono_off0, m.num_mono0, m.coef_M0, m.num_canon0, m.coef_M0_canon);
    if (m.num_interactions == 3)
        load_full_contraction("Mm_monomials", "Mm_weights", m.progm, m.mono_offm, m.num_monom, m.coef_Mm, m.num_canonm, m.coef_Mm_canon);
    {
        auto lists = detail::int_lists(file.at("M1_monomials"));
        m.prog1 = compile_polynomial(lists, m.num_lm);
        m.num_mono1 = static_cast<int>(lists.size());
        const JsonValue& weights = file.at("M1_weights");
        m.coef_M1.assign(size_t(E) * m.num_mono1 * K, 0.0);
        m.num_canon1 = kCanonPolyCount[0];
        m.coef_M1_canon.assign(size_t(E) * m.num_canon1 * K, 0.0);
        const std::vector<int> slots1 = detail::canonical_slots(lists, 0);
        for (int sl : slots1) if (sl < 0) m.poly_canonical = false;
        for (int a = 0; a < E; ++a) {
            const JsonValue& wa = weights.at(std::to_string(a));
            for (int k = 0; k < K; ++k) {
                const JsonValue& wk = wa.at(std::to_string(k));
                if (static_cast<int>(wk.size()) != m.num_mono1) throw ModelError("M1_weights row length differs from M1_monomials");
                for (int mu = 0; mu < m.num_mono1; ++mu) {
                    m.coef_M1[(size_t(a) * m.num_mono1 + m.prog1.alias[mu]) * K + k] += wk.nums[mu];
                    if (slots1[mu] >= 0) m.coef_M1_canon[(size_t(a) * m.num_canon1 + slots1[mu]) * K + k] += wk.nums[mu];
                }
            }
        }
    }
    return m;
}

}  // namespace smx
