// Test infrastructure (oracle build only; never linked into the product library).
//
// A thin extern "C" wrapper around the reference's own CPU evaluator, class MACE
// (libsymmetrix/source/mace.hpp:12-169), compiled unmodified from the reference tree.
// It exists so that Python tests and the CPU-baseline leg of the benchmark can drive the
// reference through ctypes. Nothing here re-implements reference arithmetic.
#include <cstring>
#include <exception>
#include <span>
#include <string>
#include <vector>

#include "mace.hpp"
#include "spherical_harmonic.hpp"

namespace {
thread_local std::string g_err;

std::vector<double>* field(MACE* m, const char* name) {
    const std::string s(name);
    if (s == "node_energies") return &m->node_energies;
    if (s == "node_forces") return &m->node_forces;
    if (s == "Y") return &m->Y;
    if (s == "Y_grad") return &m->Y_grad;
    if (s == "R0") return &m->R0;
    if (s == "R0_deriv") return &m->R0_deriv;
    if (s == "R1") return &m->R1;
    if (s == "R1_deriv") return &m->R1_deriv;
    if (s == "A0") return &m->A0;
    if (s == "A0_adj") return &m->A0_adj;
    if (s == "M0") return &m->M0;
    if (s == "M0_adj") return &m->M0_adj;
    if (s == "H1") return &m->H1;
    if (s == "H1_adj") return &m->H1_adj;
    if (s == "Phi1r") return &m->Phi1r;
    if (s == "Phi1") return &m->Phi1;
    if (s == "Phi1_adj") return &m->dPhi1;
    if (s == "A1") return &m->A1;
    if (s == "A1_adj") return &m->A1_adj;
    if (s == "M1") return &m->M1;
    if (s == "M1_adj") return &m->M1_adj;
    if (s == "H2") return &m->H2;
    if (s == "H2_adj") return &m->H2_adj;
    return nullptr;
}
}  // namespace

extern "C" {

const char* ref_last_error() { return g_err.c_str(); }

void* ref_create(const char* json_path) {
    try {
        return new MACE(std::string(json_path));
    } catch (const std::exception& e) {
        g_err = e.what();
        return nullptr;
    }
}

void ref_destroy(void* h) { delete static_cast<MACE*>(h); }

// out = {num_elements, num_channels, l_max, L_max, num_lelm1lm2, num_lme, has_zbl}
void ref_info(void* h, int* out, double* r_cut) {
    auto* m = static_cast<MACE*>(h);
    out[0] = m->num_elements;
    out[1] = m->num_channels;
    out[2] = m->l_max;
    out[3] = m->L_max;
    out[4] = m->num_lelm1lm2;
    out[5] = m->num_lme;
    out[6] = m->has_zbl ? 1 : 0;
    *r_cut = m->r_cut;
}

int ref_atomic_numbers(void* h, int* out, int cap) {
    auto* m = static_cast<MACE*>(h);
    const int n = static_cast<int>(m->atomic_numbers.size());
    for (int i = 0; i < n && i < cap; ++i) out[i] = m->atomic_numbers[i];
    return n;
}

// MACE::compute_node_energies_forces, libsymmetrix/source/mace.cpp:17-64
int ref_compute(void* h, int num_nodes, const int* node_types, const int* num_neigh,
                const int* neigh_indices, const int* neigh_types, const double* xyz,
                const double* r, long num_edges) {
    auto* m = static_cast<MACE*>(h);
    try {
        m->compute_node_energies_forces(
            num_nodes, std::span<const int>(node_types, num_nodes),
            std::span<const int>(num_neigh, num_nodes),
            std::span<const int>(neigh_indices, num_edges),
            std::span<const int>(neigh_types, num_edges),
            std::span<const double>(xyz, 3 * num_edges), std::span<const double>(r, num_edges));
    } catch (const std::exception& e) {
        g_err = e.what();
        return 1;
    }
    return 0;
}

// One named stage of the evaluator, with the argument subset that stage takes in the
// reference (mace.hpp:40-164). flag0/flag1 carry zero_dxyz / zero_H1_adj where they exist.
int ref_stage(void* h, const char* name, int num_nodes, const int* node_types,
              const int* num_neigh, const int* neigh_indices, const int* neigh_types,
              const double* xyz, const double* r, long num_edges, int flag0, int flag1) {
    auto* m = static_cast<MACE*>(h);
    const std::string s(name);
    auto nt = std::span<const int>(node_types, num_nodes);
    auto nn = std::span<const int>(num_neigh, num_nodes);
    auto ni = std::span<const int>(neigh_indices, num_edges);
    auto et = std::span<const int>(neigh_types, num_edges);
    auto X = std::span<const double>(xyz, 3 * num_edges);
    auto R = std::span<const double>(r, num_edges);
    try {
        if (s == "compute_Y") m->compute_Y(X);
        else if (s == "compute_R0") m->compute_R0(num_nodes, nt, nn, et, R);
        else if (s == "compute_R1") m->compute_R1(num_nodes, nt, nn, et, R);
        else if (s == "compute_A0") m->compute_A0(num_nodes, nt, nn, et);
        else if (s == "compute_A0_scaled") m->compute_A0_scaled(num_nodes, nt, nn, et, R);
        else if (s == "compute_M0") m->compute_M0(num_nodes, nt);
        else if (s == "compute_H1") m->compute_H1(num_nodes);
        else if (s == "compute_Phi1") m->compute_Phi1(num_nodes, nn, ni);
        else if (s == "compute_A1") m->compute_A1(num_nodes);
        else if (s == "compute_A1_scaled") m->compute_A1_scaled(num_nodes, nt, nn, et, R);
        else if (s == "compute_M1") m->compute_M1(num_nodes, nt);
        else if (s == "compute_H2") m->compute_H2(num_nodes, nt);
        else if (s == "compute_readouts") m->compute_readouts(num_nodes, nt);
        else if (s == "reverse_H2") m->reverse_H2(num_nodes, nt, flag1 != 0);
        else if (s == "reverse_M1") m->reverse_M1(num_nodes, nt);
        else if (s == "reverse_A1_scaled") m->reverse_A1_scaled(num_nodes, nt, nn, et, X, R, flag0 != 0);
        else if (s == "reverse_A1") m->reverse_A1(num_nodes);
        else if (s == "reverse_Phi1") m->reverse_Phi1(num_nodes, nn, ni, X, R, flag0 != 0, flag1 != 0);
        else if (s == "reverse_H1") m->reverse_H1(num_nodes);
        else if (s == "reverse_M0") m->reverse_M0(num_nodes, nt);
        else if (s == "reverse_A0_scaled") m->reverse_A0_scaled(num_nodes, nt, nn, et, X, R);
        else if (s == "reverse_A0") m->reverse_A0(num_nodes, nt, nn, et, X, R);
        else { g_err = "unknown stage " + s; return 2; }
    } catch (const std::exception& e) {
        g_err = e.what();
        return 1;
    }
    return 0;
}

// Read access to a public std::vector<double> member by name. Returns its length.
long ref_get(void* h, const char* name, const double** ptr) {
    auto* v = field(static_cast<MACE*>(h), name);
    if (!v) { g_err = std::string("unknown field ") + name; return -1; }
    *ptr = v->data();
    return static_cast<long>(v->size());
}

// Write access (the message-passing pair-style mode swaps H1 / H1_adj in and out,
// pair_symmetrix/pair_symmetrix_mace.cpp:463-471,488-490).
int ref_set(void* h, const char* name, const double* src, long n) {
    auto* v = field(static_cast<MACE*>(h), name);
    if (!v) { g_err = std::string("unknown field ") + name; return 1; }
    v->assign(src, src + n);
    return 0;
}

// The reference's closed-form real spherical harmonic (spherical_harmonic.cpp:38-43),
// exported to pin the sign/ordering convention of the sphericart restatement.
double ref_real_sph_harm_xyz(int l, int m, double x, double y, double z) {
    return real_sph_harm_xyz(l, m, x, y, z);
}

}  // extern "C"
