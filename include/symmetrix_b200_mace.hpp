// C++ facade with the shape of the reference's `class MACE`
// (libsymmetrix/source/mace.hpp:12-169), implemented on the C ABI of symmetrix_b200.h.
//
// Code written against the reference class -- the LAMMPS pair style
// (pair_symmetrix/pair_symmetrix_mace.cpp:115-164,242-748) or pybind11 lambdas
// (symmetrix/source/cpp/mace.cpp:35-243) -- compiles against this header with the include and
// the type name changed: same constructor, same public data members, same method names and
// argument lists. Differences that a caller can observe:
//   * the work happens on the GPU; the `std::vector` members are host mirrors, refreshed by
//     compute_node_energies_forces() (node_energies, node_forces) or on request (pull("H1"));
//   * stage methods use the edge arrays handed to begin() (or to the last whole evaluation):
//     call begin(...) where the reference code zero-fills node_energies / node_forces
//     (pair_symmetrix_mace.cpp:437-440), with the arrays of ALL receivers that any stage of the step will
//     use (owned atoms first). The array arguments of the stage methods are accepted and not read again;
//     their `num_nodes` argument is honoured: a stage called with another receiver count than the one in
//     effect switches the active receivers first (smx_set_active_nodes), which is what the pair style's
//     recompute branch relies on (layer 0 on nlocal + nghost receivers, layer 1 on nlocal,
//     pair_symmetrix_mace.cpp:672-697); a count beyond what begin() was given throws;
//   * errors surface as std::runtime_error carrying the library's message, like the reference's
//     exceptions (e.g. a non-JSON model file, symmetrix_calc.py:54-68).
#pragma once

#include <span>
#include <stdexcept>
#include <string>
#include <vector>

#include "symmetrix_b200.h"

namespace symmetrix_b200 {

class MACE {
public:
    explicit MACE(std::string filename, int precision = SMX_FP64, int device = 0) {
        if (smx_create(filename.c_str(), precision, device, &h_) != SMX_OK)
            throw std::runtime_error(smx_last_error(nullptr));
        smx_model_info info{};
        check(smx_info(h_, &info));
        num_elements = info.num_elements; num_channels = info.num_channels; r_cut = info.r_cut;
        l_max = info.l_max; num_lm = info.num_lm; L_max = info.L_max; num_LM = info.num_LM;
        num_lelm1lm2 = info.num_lelm1lm2; num_lme = info.num_lme; has_zbl = info.has_zbl != 0;
        atomic_numbers.resize(num_elements);
        atomic_energies.resize(num_elements);
        smx_atomic_numbers(h_, atomic_numbers.data(), num_elements);
        smx_atomic_energies(h_, atomic_energies.data(), num_elements);
    }
    ~MACE() { smx_destroy(h_); }
    MACE(const MACE&) = delete;
    MACE& operator=(const MACE&) = delete;

    // Basic model information (mace.hpp:18-25,39,112)
    int num_elements = 0, num_channels = 0;
    double r_cut = 0.0;
    int l_max = 0, num_lm = 0, L_max = 0, num_LM = 0, num_lelm1lm2 = 0, num_lme = 0;
    std::vector<int> atomic_numbers;
    std::vector<double> atomic_energies;
    bool has_zbl = false;

    // The pair style calls mace->zbl.compute_ZBL(...) by hand in its staged modes (pair_symmetrix_mace.cpp:441-444).
    struct ZBLStage {
        MACE* owner = nullptr;
        template <typename... A> void compute_ZBL(int num_nodes, A&&...) { owner->stage_on(num_nodes, "compute_ZBL"); }
    } zbl{this};

    // Host mirrors of the public vectors the callers read or swap (mace.hpp:28,104)
    std::vector<double> node_energies, node_forces, H1, H1_adj;
    std::vector<double> Hm, Hm_adj;   // features of the middle block of a three-block model (exchanged like H1 / H1_adj)

    // mace.hpp:29-36 / mace.cpp:17-64
    void compute_node_energies_forces(const int num_nodes, std::span<const int> node_types, std::span<const int> num_neigh,
                                      std::span<const int> neigh_indices, std::span<const int> neigh_types,
                                      std::span<const double> xyz, std::span<const double> r) {
        check(smx_compute(h_, num_nodes, node_types.data(), num_neigh.data(), neigh_indices.data(), neigh_types.data(),
                          xyz.data(), r.data(), static_cast<long>(r.size()), SMX_HOST));
        active_nodes_ = num_nodes;
        pull("node_energies");
        pull("node_forces");
    }

    // Sets the edge arrays for the stage methods and zero-fills node_energies / node_forces on the device.
    void begin(const int num_nodes, std::span<const int> node_types, std::span<const int> num_neigh,
               std::span<const int> neigh_indices, std::span<const int> neigh_types, std::span<const double> xyz,
               std::span<const double> r) {
        check(smx_begin(h_, num_nodes, node_types.data(), num_neigh.data(), neigh_indices.data(), neigh_types.data(), xyz.data(),
                        r.data(), static_cast<long>(r.size()), SMX_HOST));
        active_nodes_ = num_nodes;
    }

    // Stage methods (mace.hpp:40-164) with the reference's argument lists: `num_nodes` selects the active receivers
    // (see the header comment), the array arguments are those already given to begin() and are not read again.
    template <typename... A> void compute_Y(A&&...) { stage("compute_Y"); }
    template <typename... A> void compute_R0(int num_nodes, A&&...) { stage_on(num_nodes, "compute_R0"); }
    template <typename... A> void compute_R1(int num_nodes, A&&...) { stage_on(num_nodes, "compute_R1"); }
    template <typename... A> void compute_A0(int num_nodes, A&&...) { stage_on(num_nodes, "compute_A0"); }
    template <typename... A> void compute_A0_scaled(int num_nodes, A&&...) { stage_on(num_nodes, "compute_A0_scaled"); }
    template <typename... A> void compute_M0(int num_nodes, A&&...) { stage_on(num_nodes, "compute_M0"); }
    template <typename... A> void compute_H1(int num_nodes, A&&...) { stage_on(num_nodes, "compute_H1"); }
    template <typename... A> void compute_A1(int num_nodes, A&&...) { stage_on(num_nodes, "compute_A1"); }
    template <typename... A> void compute_A1_scaled(int num_nodes, A&&...) { stage_on(num_nodes, "compute_A1_scaled"); }
    template <typename... A> void compute_M1(int num_nodes, A&&...) { stage_on(num_nodes, "compute_M1"); }
    template <typename... A> void compute_H2(int num_nodes, A&&...) { stage_on(num_nodes, "compute_H2"); }
    template <typename... A> void compute_readouts(int num_nodes, A&&...) { stage_on(num_nodes, "compute_readouts"); }
    template <typename... A> void reverse_M1(int num_nodes, A&&...) { stage_on(num_nodes, "reverse_M1"); }
    template <typename... A> void reverse_A1(int num_nodes, A&&...) { stage_on(num_nodes, "reverse_A1"); }
    template <typename... A> void reverse_H1(int num_nodes, A&&...) { stage_on(num_nodes, "reverse_H1"); }
    template <typename... A> void reverse_M0(int num_nodes, A&&...) { stage_on(num_nodes, "reverse_M0"); }
    template <typename... A> void reverse_A0(int num_nodes, A&&...) { stage_on(num_nodes, "reverse_A0"); }
    template <typename... A> void reverse_A0_scaled(int num_nodes, A&&...) { stage_on(num_nodes, "reverse_A0_scaled"); }
    // The sender index array decides which rows of H1 are gathered (mace.hpp:117); here it is the one given to begin().
    void compute_Phi1(const int num_nodes, std::span<const int>, std::span<const int>) { stage_on(num_nodes, "compute_Phi1"); }
    void reverse_Phi1(const int num_nodes, std::span<const int>, std::span<const int>, std::span<const double>, std::span<const double>,
                      bool zero_dxyz = true, bool zero_H1_adj = true) { stage_on(num_nodes, "reverse_Phi1", zero_dxyz, zero_H1_adj); }
    void reverse_H2(const int num_nodes, std::span<const int>, bool zero_H1_adj = true) { stage_on(num_nodes, "reverse_H2", true, zero_H1_adj); }
    void reverse_A1_scaled(const int num_nodes, std::span<const int>, std::span<const int>, std::span<const int>, std::span<const double>,
                           std::span<const double>, bool zero_dxyz = true) { stage_on(num_nodes, "reverse_A1_scaled", zero_dxyz, true); }

    // Middle interaction block of a model whose file says "num_interactions": 3. The reference has no counterpart (its
    // models have exactly two blocks, extract_mace_data.py:70-71); the stages take the place of a second
    // compute_Phi1 ... compute_H2 group with every (L, M) kept, called between compute_H1 and compute_R1 / compute_Phi1,
    // and their reverses between reverse_Phi1 and reverse_H1. Arrays: "Phim", "Am", "Mm", "Hm" and "*_adj".
    void compute_Rm() { stage("compute_Rm"); }
    void compute_Phim() { stage("compute_Phim"); }
    void compute_Am() { stage("compute_Am"); }
    void compute_Mm() { stage("compute_Mm"); }
    void compute_Hm() { stage("compute_Hm"); }
    void reverse_Hm() { stage("reverse_Hm"); }
    void reverse_Mm() { stage("reverse_Mm"); }
    void reverse_Am() { stage("reverse_Am"); }
    void reverse_Phim(bool zero_dxyz = true, bool zero_H1_adj = true) { stage("reverse_Phim", zero_dxyz, zero_H1_adj); }

    // Device <-> host mirrors: pull("H1") after compute_H1, push("H1") after a forward halo exchange, etc.
    std::vector<double>& pull(const std::string& name) {
        std::vector<double>& v = mirror(name);
        long n = 0;
        check(smx_get_array(h_, name.c_str(), nullptr, 0, &n, SMX_HOST));
        v.resize(static_cast<size_t>(n));
        if (n) check(smx_get_array(h_, name.c_str(), v.data(), n, &n, SMX_HOST));
        return v;
    }
    void push(const std::string& name) {
        const std::vector<double>& v = mirror(name);
        check(smx_set_array(h_, name.c_str(), v.data(), static_cast<long>(v.size()), SMX_HOST));
    }
    // f[i] -= nf_ij, f[j] += nf_ij, virial, energy (pair_symmetrix_mace.cpp:324-368) on the device.
    void reduce_forces(int num_rows, double* atom_forces, double* virial6, double* energy) {
        check(smx_reduce_forces(h_, num_rows, atom_forces, virial6, energy, SMX_HOST));
    }
    // Receiver count of the stage calls that follow. The reference passes `num_nodes` to every stage; its recompute
    // branch (pair_symmetrix_mace.cpp:551-748) runs layer 0 on nlocal + nghost receivers and layer 1 on nlocal. Here the
    // edge set is given once to begin() with all receivers (owned first); restrict_nodes starts an evaluation on the
    // first `num_nodes`, set_active_nodes changes the count in the middle of one and keeps the accumulated outputs.
    long restrict_nodes(int num_nodes) { long e = 0; check(smx_restrict_nodes(h_, num_nodes, &e)); active_nodes_ = num_nodes; return e; }
    long set_active_nodes(int num_nodes) { long e = 0; check(smx_set_active_nodes(h_, num_nodes, &e)); active_nodes_ = num_nodes; return e; }
    // Grow "H1" / "H1_adj" to `rows` feature rows (ghost rows appended, zero-filled), as the pair style resizes its H1
    // vector to nlocal + nghost rows before forward_comm (pair_symmetrix_mace.cpp:463-464).
    void resize_rows(const std::string& name, int rows) { check(smx_resize_rows(h_, name.c_str(), rows)); }
    smx_handle handle() const { return h_; }

private:
    smx_handle h_ = nullptr;
    std::vector<double> scratch_;
    void check(int status) const {
        if (status != SMX_OK) throw std::runtime_error(smx_last_error(h_));
    }
    int active_nodes_ = -1;       // receiver count in effect (-1: taken from the library at the first staged call)
    void stage(const char* name, bool zero_dxyz = true, bool zero_H1_adj = true) {
        check(smx_stage(h_, name, zero_dxyz ? 1 : 0, zero_H1_adj ? 1 : 0));
    }
    // A stage on `num_nodes` receivers: switches the active receivers when the count differs from the one in effect.
    void stage_on(int num_nodes, const char* name, bool zero_dxyz = true, bool zero_H1_adj = true) {
        if (active_nodes_ < 0) check(smx_active_counts(h_, &active_nodes_, nullptr, nullptr));
        if (num_nodes != active_nodes_) set_active_nodes(num_nodes);
        stage(name, zero_dxyz, zero_H1_adj);
    }
    std::vector<double>& mirror(const std::string& name) {
        if (name == "node_energies") return node_energies;
        if (name == "node_forces") return node_forces;
        if (name == "H1") return H1;
        if (name == "H1_adj") return H1_adj;
        if (name == "Hm") return Hm;
        if (name == "Hm_adj") return Hm_adj;
        throw std::runtime_error("no host mirror for '" + name + "'");
    }
};

}  // namespace symmetrix_b200
