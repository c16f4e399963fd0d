// Host side of the evaluator: class template Evaluator<T>, instantiated for float (evaluator_f32.cu) and double
// (evaluator_f64.cu); the extern "C" entry points declared in include/symmetrix_b200.h are in capi.cu.
// Mirrors the stage structure of the reference's `class MACE` (libsymmetrix/source/mace.hpp:12-169):
// one method per compute_*/reverse_* stage, run in the order of MACE::compute_node_energies_forces
// (mace.cpp:17-64). There is no CPU path: creation fails when no CUDA device is usable.
#pragma once
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <tuple>
#include <vector>

#include <cub/cub.cuh>
#include <nvtx3/nvToolsExt.h>

#include "../../include/symmetrix_b200.h"
#include "common.cuh"
#include "kernels.cuh"
#include "gemm_tcgen05.cuh"
#include <type_traits>

#include "model.hpp"
#include "evaluator_base.hpp"
#include "neighbors.cuh"
#include "nccl_transport.hpp"

namespace smx {

template <typename T>
static std::vector<T> cast_vec(const std::vector<double>& v) {
    std::vector<T> o(v.size());
    for (size_t i = 0; i < v.size(); ++i) o[i] = static_cast<T>(v[i]);
    return o;
}

// Spline tables for the device: rows of 4*K values per (pair, bin, function block). float keeps the host
// order [K][4]; double splits every row into [2][K][2] so that both 16-byte loads of a warp are contiguous
// (see load_coef).
template <typename T>
static std::vector<T> spline_rows(const std::vector<double>& v, int K) {
    if constexpr (std::is_same<T, float>::value) {
        return cast_vec<T>(v);
    } else {
        std::vector<T> o(v.size());
        const size_t row = static_cast<size_t>(4) * K;
        for (size_t r0 = 0; r0 + row <= v.size(); r0 += row)
            for (int k = 0; k < K; ++k) {
                o[r0 + 2 * k] = v[r0 + 4 * k];
                o[r0 + 2 * k + 1] = v[r0 + 4 * k + 1];
                o[r0 + 2 * K + 2 * k] = v[r0 + 4 * k + 2];
                o[r0 + 2 * K + 2 * k + 1] = v[r0 + 4 * k + 3];
            }
        return o;
    }
}

// NVTX range around a stage or a whole evaluation (visible in Nsight Systems timelines; costs nothing when no tool is attached).
struct NvtxRange {
    explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
    NvtxRange(const NvtxRange&) = delete;
    NvtxRange& operator=(const NvtxRange&) = delete;
};

struct CastToLL {
    __host__ __device__ long long operator()(const int& v) const { return static_cast<long long>(v); }
};

template <typename T>
class Evaluator final : public EvaluatorBase {
public:
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr, evt0 = nullptr, evt1 = nullptr;
    std::vector<cudaEvent_t> stage_events;
    int num_sms = 148;
    int max_dynamic_smem = 0;     // sharedMemPerBlockOptin of the device

    // model tables on the device
    DevBuf<T> coef0, coef1, H0_w, A0_w, H1_w, A1_w, H2_w_H1, H2_w_M1, ro1, ro2_w1, ro2_w2, coefM0, coefM1;
    DevBuf<T> coef0_folded;       // layer-0 table with H0 and the per-type channel mix folded in (see fold_layer0_kernel)
    bool fold_a0 = false;
    DevBuf<T> coefm, Am_w, Hm_w, Hm_res, ro_m, coefMm;    // middle interaction block (models with three blocks)
    DevBuf<int> progm, progm_off, progm_cnt, monom_off;
    bool poly_fixed = false;      // coefM0 / coefM1 hold the canonical order and the straight-line kernels are used
    DevBuf<double> E0, zbl_radii, A0_spl, A1_spl;
    DevBuf<int> zbl_numbers;
    DevBuf<int> prog0, prog0_off, prog0_cnt, mono0_off, prog1, prog1_off, prog1_cnt, mono1_off;
    SplineMeta sm{};

    // current edge set
    int N = 0;
    long E = 0;
    int N_built = 0;              // receivers of the edge set as given or built; N <= N_built are active
    int h1_rows = 0;
    int hm_rows = 0;              // rows of Hm / Hm_adj (three-block models), as h1_rows for H1
    bool have_edges = false;
    DevBuf<int> in_node_types, in_num_neigh, in_neigh_indices, in_neigh_types, in_shifts;
    DevBuf<double> in_xyz, in_r;
    const int *node_types = nullptr, *num_neigh = nullptr, *neigh_indices = nullptr, *neigh_types = nullptr;
    const double *xyz = nullptr, *r = nullptr;
    DevBuf<long long> first_neigh, in_ptr;
    DevBuf<int> perm, sorted_types, type_seg, iota, in_edge, sorted_senders;
    DevBuf<int> work_sched, work_counts, work_item_ptr, work_n_items;    // work distribution of the edge kernels (see work_first)
    DevBuf<int4> work_items;
    DevBuf<unsigned char> cub_tmp;
    DevBuf<int> halo_iota, halo_rows, halo_pos;    // positions of an unpack-add list grouped by destination row
    // smx_halo_cache_lists: groupings kept per (address, length) of an index list, for callers whose lists stay put
    struct HaloGrouping { std::unique_ptr<DevBuf<int>> rows, pos; };
    std::map<std::pair<const int*, int>, HaloGrouping> halo_groupings;
    bool halo_cache = false;
    int sender_rows = -1;
    std::vector<long long> first_host;   // host copy of first_neigh for restrict_nodes (valid until the edge set changes)
    bool first_host_valid = false;

    // per-call arrays
    DevBuf<T> Phi0, A0, A0_adj, Phi0_adj, M0, M0_adj, H1, H1_adj, Phi1, dPhi1, A1, A1_adj, M1, M1_adj, H2, H2_adj, Hmsg;
    DevBuf<T> Phim, dPhim, Am, Am_adj, Mm, Mm_adj, Hm, Hm_adj;
    DevBuf<double> node_energies, node_forces, scratch_d, partials, out7, atom_f;
    // GEMM problem lists travel through a pinned host ring and a device ring, so launches need no host synchronisation;
    // the rings hold far more entries than one evaluation uses (a slot is reused only thousands of launches later)
    static constexpr size_t kProblemRing = 8192;
    GemmProblem<T>* host_ring = nullptr;
    DevBuf<GemmProblem<T>> dev_ring;
    size_t ring_pos = 0;
    bool own_stream = true;
    DevBuf<int> kernel_status;    // non-zero if a bounded mbarrier wait ran out (1, 2: tcgen05 GEMM; 3, 4: staged tensor-product reverse)
    bool staged_reverse = false;  // spline rows of the tensor-product reverse through bulk copies into shared memory
                                  // (SMX_TP_STAGED=1; measured equal in float64 and 15 % slower in float32 on B200)
    // Run-time radial mode (SMX_RADIAL=mlp, float32, two-block models whose file carries the x_radial_* keys): the radial
    // functions of block 1 come from the un-splined network -- hidden layers per edge (radial_hidden_kernel), last layer
    // as a tensor-core GEMM over all edges -- instead of the spline tables.
    bool radial_mlp = false;
    bool radial_lowrank = false;          // SMX_RADIAL=lowrank: hidden activations from the tabulated last hidden layer (inside the
                                          // fused kernels) instead of radial_hidden_kernel; the last layer on the tensor cores as above
    DevBuf<float> rn_basis;
    bool radial_hidden_valid = false;     // x3 / dx3 hold the hidden activations of the current active edge set
    DevBuf<float> rn_w_first, rn_w_hidden, rn_w_last, rn_pair_scale, rn_x, rn_dx;
    DevBuf<T> R_edge, Rd_edge;
    DevBuf<unsigned char> rn_tiles;       // float16 weight tiles of the last layer, one per path (radial_prepare_tiles_kernel)
    bool radial_fused = true;             // SMX_RADIAL_FUSED=0: last layer as a separate GEMM into per-edge arrays also in the forward pass
    bool radial_in_kernel = false;        // set around the launch of the fused forward kernel
    int tmem_min_blocks = 3;      // SMX_TP_TMEM_BLOCKS: 2, 3 or 4 resident CTAs per SM for that kernel (3 measured best on B200)
    bool tmem_reverse = true;     // float64 tensor-product reverse with the receiver adjoint in tensor memory (SMX_TP_TMEM=0: in registers)
    bool type_order = true;       // edge kernels walk the receivers in element-type order (SMX_TYPE_ORDER=0: natural order)
    bool waits_in_flight = false; // a kernel with bounded waits has been launched since the last status check
    bool use_tc5 = false;
    bool gemm_async = true;       // float64 GEMMs with cp.async tile loads (SMX_GEMM=mma: the register-staged kernel)
    std::map<std::tuple<const void*, int, int, int, int>, std::unique_ptr<DevBuf<float>>> weight_images;
    cudaStream_t own_stream_handle = nullptr;
    cudaStream_t copy_stream = nullptr;       // host -> device copies of the geometry (see begin)
    cudaEvent_t copy_ready = nullptr, copy_done = nullptr;
    NeighborBuilder nb;

    explicit Evaluator(HostModel&& m, int dev) {
        model = std::move(m);
        device = dev;
        precision = sizeof(T) == 4 ? 32 : 64;
        SMX_CUDA(cudaSetDevice(dev));
        SMX_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
        SMX_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&host_ring), kProblemRing * sizeof(GemmProblem<T>), cudaHostAllocDefault));
        dev_ring.resize(kProblemRing, stream);
        kernel_status.resize(2, stream);      // [0] error code of a wait that ran out, [1] test switch (see gemm_rows_tcgen05_kernel)
        kernel_status.zero(stream);
        if (const char* t = std::getenv("SMX_TP_STAGED")) staged_reverse = std::string(t) != "0";
        if (const char* t = std::getenv("SMX_TYPE_ORDER")) type_order = std::string(t) != "0";
        if (const char* t = std::getenv("SMX_TP_TMEM")) tmem_reverse = std::string(t) != "0";
        if (const char* t = std::getenv("SMX_TP_TMEM_BLOCKS")) tmem_min_blocks = std::max(2, std::min(4, std::atoi(t)));
        if (const char* t = std::getenv("SMX_RADIAL")) {
            const std::string mode(t);
            if (mode == "mlp" || mode == "lowrank") {
                if (sizeof(T) != 4) throw UnsupportedError("SMX_RADIAL=" + mode + " is a float32 mode (the float64 path reproduces the reference's splines)");
                if (!model.rmlp1.present) throw UnsupportedError("SMX_RADIAL=" + mode + " needs the x_radial_* keys in the model file");
                if (model.num_interactions != 2) throw UnsupportedError("SMX_RADIAL=" + mode + " supports two-block models");
                radial_mlp = true;
                if (const char* f = std::getenv("SMX_RADIAL_FUSED")) radial_fused = std::string(f) != "0";
                if (mode == "lowrank") {
                    if (model.rmlp1.basis_coef.empty()) throw UnsupportedError("SMX_RADIAL=lowrank needs the x_radial_basis_* keys in the model file");
                    if (model.K > 128 || model.L_max > 1 || model.rmlp1.hidden > kRnHidden)
                        throw UnsupportedError("SMX_RADIAL=lowrank supports up to 128 channels, L_max <= 1 and a hidden width up to 64");
                    radial_lowrank = true;
                    radial_fused = true;
                }
            } else if (mode != "spline" && !mode.empty()) {
                throw ArgError("SMX_RADIAL must be 'spline', 'mlp' or 'lowrank'");
            }
        }
        if (const char* g = std::getenv("SMX_GEMM")) gemm_async = std::string(g) != "mma";
        if constexpr (sizeof(T) == 4) {
            // float32 GEMMs run on tcgen05 unless SMX_GEMM=mma asks for the mma.sync kernel
            const char* g = std::getenv("SMX_GEMM");
            use_tc5 = !(g && std::string(g) == "mma");
            SMX_CUDA(cudaFuncSetAttribute(gemm_rows_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTc5SmemBytes));
        }
        SMX_CUDA(cudaEventCreate(&ev0));
        SMX_CUDA(cudaEventCreate(&ev1));
        SMX_CUDA(cudaEventCreate(&evt0));
        SMX_CUDA(cudaEventCreate(&evt1));
        cudaDeviceProp prop{};
        SMX_CUDA(cudaGetDeviceProperties(&prop, dev));
        num_sms = prop.multiProcessorCount;
        max_dynamic_smem = static_cast<int>(prop.sharedMemPerBlockOptin);
        upload_model();
    }
    ~Evaluator() override {
        cudaSetDevice(device);
        if (stream) cudaStreamSynchronize(stream);
        if (ev0) cudaEventDestroy(ev0);
        if (ev1) cudaEventDestroy(ev1);
        if (evt0) cudaEventDestroy(evt0);
        if (evt1) cudaEventDestroy(evt1);
        for (auto e : stage_events) cudaEventDestroy(e);
        if (comm) NcclApi::get().CommDestroy(comm);
        if (copy_stream) { cudaStreamSynchronize(copy_stream); cudaStreamDestroy(copy_stream); cudaEventDestroy(copy_ready); cudaEventDestroy(copy_done); }
        if (host_ring) cudaFreeHost(host_ring);
        if (!own_stream && own_stream_handle) cudaStreamDestroy(own_stream_handle);
        if (stream && own_stream) cudaStreamDestroy(stream);
    }

    void upload_model() {
        const HostModel& m = model;
        coef0.upload(spline_rows<T>(m.coef0, m.K), stream);
        coef1.upload(spline_rows<T>(m.coef1, m.K), stream);

        H0_w.upload(cast_vec<T>(m.H0_w), stream);
        A0_w.upload(cast_vec<T>(m.A0_w), stream);
        {
            // Folded layer-0 table (SMX_A0_FOLD=0 keeps the two-step form): E^2 instead of E (E + 1) / 2 pair tables, so only
            // for models with few element types
            const char* f = std::getenv("SMX_A0_FOLD");
            fold_a0 = !(f && std::string(f) == "0") && m.num_elements <= 16 && m.K <= 1024;
            const size_t bins = static_cast<size_t>(m.num_bins);
            const size_t pairs = static_cast<size_t>(m.num_elements) * (m.num_elements + 1) / 2;
            if (fold_a0 && m.coef0.size() == pairs * bins * 16 * m.K && m.A0_w.size() == static_cast<size_t>(m.num_elements) * 4 * m.K * m.K) {
                DevBuf<double> d_coef, d_h0, d_w;
                d_coef.upload(m.coef0, stream); d_h0.upload(m.H0_w, stream); d_w.upload(m.A0_w, stream);
                const size_t rows = static_cast<size_t>(m.num_elements) * m.num_elements * bins * 4;
                coef0_folded.resize(rows * 4 * m.K, stream);
                fold_layer0_kernel<T><<<static_cast<unsigned>(rows), std::min(256, ((m.K + 31) / 32) * 32), static_cast<size_t>(4) * m.K * sizeof(double), stream>>>(
                    m.num_elements, static_cast<int>(bins), m.K, d_coef.p, d_h0.p, d_w.p, coef0_folded.p);
                check_launch("fold_layer0_kernel");
                SMX_CUDA(cudaStreamSynchronize(stream));      // the temporaries are freed on leaving this scope
            } else {
                fold_a0 = false;
            }
        }
        H1_w.upload(cast_vec<T>(m.H1_w), stream);
        A1_w.upload(cast_vec<T>(m.A1_w), stream);
        H2_w_H1.upload(cast_vec<T>(m.H2_w_H1), stream);
        H2_w_M1.upload(cast_vec<T>(m.H2_w_M1), stream);
        ro1.upload(cast_vec<T>(m.ro1), stream);
        ro2_w1.upload(cast_vec<T>(m.ro2_w1), stream);
        ro2_w2.upload(cast_vec<T>(m.ro2_w2), stream);
        poly_fixed = m.poly_canonical;
        coefM0.upload(cast_vec<T>(poly_fixed ? m.coef_M0_canon : m.coef_M0), stream);
        coefM1.upload(cast_vec<T>(poly_fixed ? m.coef_M1_canon : m.coef_M1), stream);
        if (m.num_interactions == 3) {
            coefm.upload(spline_rows<T>(m.coefm, m.K), stream);
            Am_w.upload(cast_vec<T>(m.Am_w), stream);
            Hm_w.upload(cast_vec<T>(m.Hm_w), stream);
            Hm_res.upload(cast_vec<T>(m.Hm_res), stream);
            ro_m.upload(cast_vec<T>(m.ro_m), stream);
            coefMm.upload(cast_vec<T>(poly_fixed ? m.coef_Mm_canon : m.coef_Mm), stream);
            std::vector<int> words, offs, counts;
            for (const auto& p : m.progm) {
                offs.push_back(static_cast<int>(words.size()));
                counts.push_back(static_cast<int>(p.words.size()) - kPolyPrefetch);
                words.insert(words.end(), p.words.begin(), p.words.end());
            }
            progm.upload(words, stream);
            progm_off.upload(offs, stream);
            progm_cnt.upload(counts, stream);
            monom_off.upload(std::vector<int>(m.mono_offm.begin(), m.mono_offm.end() - 1), stream);
        }
        if (radial_mlp) {
            rn_w_first.upload(cast_vec<float>(m.rmlp1.w_first), stream);
            rn_w_hidden.upload(cast_vec<float>(m.rmlp1.w_hidden), stream);
            rn_w_last.upload(cast_vec<float>(m.rmlp1.w_last), stream);
            rn_pair_scale.upload(cast_vec<float>(m.rmlp1.pair_scale), stream);
            if (radial_lowrank) rn_basis.upload(cast_vec<float>(m.rmlp1.basis_coef), stream);
            if (m.K <= 128 && m.L_max <= 1 && m.rmlp1.hidden <= kRnHidden) {
                rn_tiles.resize(static_cast<size_t>(m.tp.P) * kRnTileBytes, stream);
                radial_prepare_tiles_kernel<<<64, 256, 0, stream>>>(rn_w_last.p, m.rmlp1.hidden, m.K, m.tp.P, rn_tiles.p);
                check_launch("radial_prepare_tiles_kernel");
            }
        }
        E0.upload(m.atomic_energies, stream);
        if (m.has_zbl) { zbl_radii.upload(m.zbl_covalent_radii, stream); zbl_numbers.upload(m.atomic_numbers, stream); }
        if (m.A0_scaled) A0_spl.upload(m.A0_spline_coef, stream);
        if (m.A1_scaled) A1_spl.upload(m.A1_spline_coef, stream);
        {
            // per output: [first word, number of operations to execute (without the trailing prefetch padding)]
            std::vector<int> words, offs, counts;
            for (const auto& p : m.prog0) {
                offs.push_back(static_cast<int>(words.size()));
                counts.push_back(static_cast<int>(p.words.size()) - kPolyPrefetch);
                words.insert(words.end(), p.words.begin(), p.words.end());
            }
            prog0.upload(words, stream);
            prog0_off.upload(offs, stream);
            prog0_cnt.upload(counts, stream);
            mono0_off.upload(std::vector<int>(m.mono_off0.begin(), m.mono_off0.end() - 1), stream);
            prog1.upload(m.prog1.words, stream);
            prog1_off.upload(std::vector<int>{0}, stream);
            prog1_cnt.upload(std::vector<int>{static_cast<int>(m.prog1.words.size()) - kPolyPrefetch}, stream);
            mono1_off.upload(std::vector<int>{0}, stream);
        }
        sm.h = m.spline_h;
        sm.num_bins = m.num_bins;
        sm.num_elements = m.num_elements;
        SMX_CUDA(cudaStreamSynchronize(stream));
        // the host copies of the big tables are no longer needed
        model.coef0.clear(); model.coef0.shrink_to_fit();
        model.coef1.clear(); model.coef1.shrink_to_fit();
        model.coef_M0.clear(); model.coef_M0.shrink_to_fit();
        model.coef_M0_canon.clear(); model.coef_M0_canon.shrink_to_fit();
    }

    // ------------------------------------------------------------------ launch helpers
    template <typename Kern>
    int persistent_grid(Kern kern, int block, size_t smem, long long work_items) {
        int per_sm = 1;
        SMX_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, block, smem));
        if (per_sm < 1) per_sm = 1;
        long long g = static_cast<long long>(num_sms) * per_sm;
        if (g > work_items) g = work_items;
        return g < 1 ? 1 : static_cast<int>(g);
    }
    void check_launch(const char* what) {
        cudaError_t err = cudaGetLastError();
        if (err != cudaSuccess) throw CudaError(std::string(what) + ": " + cudaGetErrorString(err));
        launches += 1;
    }
    int channel_block() const { return std::min(kChannelBlock, ((model.K + 31) / 32) * 32); }

    // ------------------------------------------------------------------ edge set
    template <typename U>
    const U* stage_input(const U* src, size_t count, DevBuf<U>& buf, int mem_space) {
        if (mem_space == SMX_DEVICE) return src;
        buf.resize(count, stream);
        if (count) SMX_CUDA(cudaMemcpyAsync(buf.p, src, count * sizeof(U), cudaMemcpyHostToDevice, stream));
        return buf.p;
    }

    void begin(int n_nodes, const int* nt, const int* nn, const int* ni, const int* et, const double* x, const double* rr,
               long n_edges, int mem_space) override {
        if (n_nodes < 0 || n_edges < 0) throw ArgError("negative size");
        if (n_nodes > 0 && (!nt || !nn)) throw ArgError("null node array");
        if (n_edges > 0 && (!ni || !et || !x || !rr)) throw ArgError("null edge array");
        if (mem_space != SMX_HOST && mem_space != SMX_DEVICE) throw ArgError("mem_space must be SMX_HOST or SMX_DEVICE");
        SMX_CUDA(cudaSetDevice(device));
        node_types = stage_input(nt, n_nodes, in_node_types, mem_space);
        num_neigh = stage_input(nn, n_nodes, in_num_neigh, mem_space);
        neigh_indices = stage_input(ni, n_edges, in_neigh_indices, mem_space);
        neigh_types = stage_input(et, n_edges, in_neigh_types, mem_space);
        if (mem_space == SMX_HOST && n_edges > 0) {
            // The geometry (4/5 of the bytes) travels on a second stream while the index arrays of the edge set (CSR offsets,
            // type order, work items: they need only the integer arrays) are built on the evaluator's stream.
            if (!copy_stream) {
                SMX_CUDA(cudaStreamCreateWithFlags(&copy_stream, cudaStreamNonBlocking));
                SMX_CUDA(cudaEventCreateWithFlags(&copy_ready, cudaEventDisableTiming));
                SMX_CUDA(cudaEventCreateWithFlags(&copy_done, cudaEventDisableTiming));
            }
            in_xyz.resize(3 * static_cast<size_t>(n_edges), stream);
            in_r.resize(n_edges, stream);
            SMX_CUDA(cudaEventRecord(copy_ready, stream));              // kernels of the previous evaluation may still read the buffers
            SMX_CUDA(cudaStreamWaitEvent(copy_stream, copy_ready, 0));
            SMX_CUDA(cudaMemcpyAsync(in_xyz.p, x, 3 * static_cast<size_t>(n_edges) * sizeof(double), cudaMemcpyHostToDevice, copy_stream));
            SMX_CUDA(cudaMemcpyAsync(in_r.p, rr, static_cast<size_t>(n_edges) * sizeof(double), cudaMemcpyHostToDevice, copy_stream));
            SMX_CUDA(cudaEventRecord(copy_done, copy_stream));
            xyz = in_xyz.p;
            r = in_r.p;
            N_built = n_nodes;
            adopt_edges(n_nodes, n_edges);
            ensure_sender_lists(N);                                     // the sender-sorted edge list as well (needs neigh_indices only)
            SMX_CUDA(cudaStreamWaitEvent(stream, copy_done, 0));
            return;
        }
        xyz = stage_input(x, 3 * static_cast<size_t>(n_edges), in_xyz, mem_space);
        r = stage_input(rr, n_edges, in_r, mem_space);
        N_built = n_nodes;
        adopt_edges(n_nodes, n_edges);
    }

    // Derived index arrays of the current edge set: CSR offsets and nodes sorted by element type.
    // `keep`: change the active receivers in the middle of an evaluation -- the outputs accumulated so far and the
    // feature rows beyond the active nodes stay as they are.
    void adopt_edges(int n_nodes, long n_edges, bool keep = false, bool rescan = true) {
        N = n_nodes;
        E = n_edges;
        if (!keep) { h1_rows = N; hm_rows = N; }
        sender_rows = -1;
        have_edges = true;
        radial_hidden_valid = false;
        if (rescan) {
            first_host_valid = false;
            // offsets of all receivers; a restricted set uses a prefix of this scan (entry n = edges of the first n)
            first_neigh.resize(static_cast<size_t>(N) + 1, stream);
            if (N > 0) {
                cub::TransformInputIterator<long long, CastToLL, const int*> it(num_neigh, CastToLL());
                size_t bytes = 0;
                SMX_CUDA(cub::DeviceScan::ExclusiveSum(nullptr, bytes, it, first_neigh.p, N, stream));
                cub_tmp.resize(bytes, stream);
                SMX_CUDA(cub::DeviceScan::ExclusiveSum(cub_tmp.p, bytes, it, first_neigh.p, N, stream));
                launches += 1;
            }
            const long long total = E;
            SMX_CUDA(cudaMemcpyAsync(first_neigh.p + N, &total, sizeof(long long), cudaMemcpyHostToDevice, stream));
        }
        // nodes sorted by element type (stable), and the segment of each type
        perm.resize(N, stream);
        sorted_types.resize(N, stream);
        type_seg.resize(model.num_elements + 1, stream);
        if (N > 0) {
            iota.resize(N, stream);
            iota_kernel<<<std::min(1024, (N + 255) / 256), 256, 0, stream>>>(N, iota.p);
            check_launch("iota");
            int bits = 1;
            while ((1 << bits) < model.num_elements) ++bits;
            size_t bytes = 0;
            SMX_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, bytes, node_types, sorted_types.p, iota.p, perm.p, N, 0, bits, stream));
            cub_tmp.resize(bytes, stream);
            SMX_CUDA(cub::DeviceRadixSort::SortPairs(cub_tmp.p, bytes, node_types, sorted_types.p, iota.p, perm.p, N, 0, bits, stream));
            launches += 1;
        }
        segment_offsets_int_kernel<<<1, 128, 0, stream>>>(N, sorted_types.p, model.num_elements, type_seg.p);
        check_launch("type segments");
        // work items of the reverse edge kernels: (receiver, batch of its edges) in the order the receivers are walked
        work_sched.resize(2, stream);
        work_sched.zero(stream);
        work_n_items.resize(1, stream);
        work_n_items.zero(stream);
        work_counts.resize(static_cast<size_t>(N) + 1, stream);
        work_item_ptr.resize(static_cast<size_t>(N) + 1, stream);
        work_items.resize(static_cast<size_t>(N) + static_cast<size_t>(E) / kEdgeBatch + 1, stream);
        if (N > 0) {
            const int* order = type_order ? perm.p : nullptr;
            work_items_count_kernel<<<(N + 255) / 256, 256, 0, stream>>>(N, order, first_neigh.p, work_counts.p);
            check_launch("work_items_count_kernel");
            size_t bytes = 0;
            SMX_CUDA(cub::DeviceScan::ExclusiveSum(nullptr, bytes, work_counts.p, work_item_ptr.p, N, stream));
            cub_tmp.resize(bytes, stream);
            SMX_CUDA(cub::DeviceScan::ExclusiveSum(cub_tmp.p, bytes, work_counts.p, work_item_ptr.p, N, stream));
            launches += 1;
            work_items_fill_kernel<<<(N + 255) / 256, 256, 0, stream>>>(N, order, first_neigh.p, work_item_ptr.p, work_items.p, work_n_items.p);
            check_launch("work_items_fill_kernel");
        }
        // outputs the caller zero-fills in the reference (mace.cpp:27-30)
        if (keep) {
            // the arrays only ever grow and were zero-filled at their largest extent when the step began
            node_energies.resize(N, stream, true);
            node_forces.resize(3 * static_cast<size_t>(E), stream, true);
            return;
        }
        node_energies.resize(N, stream);
        node_energies.zero(stream);
        node_forces.resize(3 * static_cast<size_t>(E), stream);
        node_forces.zero(stream);
    }

    // Edges grouped by sender row (stable in edge order), for the atomic-free scatters.
    void ensure_sender_lists(int rows) {
        if (sender_rows == rows) return;
        in_ptr.resize(static_cast<size_t>(rows) + 1, stream);
        in_edge.resize(E, stream);
        sorted_senders.resize(E, stream);
        if (E > 0) {
            if (E > 0x7fffffffL) throw UnsupportedError("more than 2^31 edges in one call");
            iota.resize(E, stream);
            iota_kernel<<<std::min<long>(4096, (E + 255) / 256), 256, 0, stream>>>(static_cast<int>(E), iota.p);
            check_launch("iota");
            int bits = 1;
            while ((1LL << bits) < rows) ++bits;
            size_t bytes = 0;
            SMX_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, bytes, neigh_indices, sorted_senders.p, iota.p, in_edge.p,
                                                     static_cast<int>(E), 0, bits, stream));
            cub_tmp.resize(bytes, stream);
            SMX_CUDA(cub::DeviceRadixSort::SortPairs(cub_tmp.p, bytes, neigh_indices, sorted_senders.p, iota.p, in_edge.p,
                                                     static_cast<int>(E), 0, bits, stream));
            launches += 1;
        }
        segment_offsets_kernel<<<std::min(1024, (rows + 256) / 256), 256, 0, stream>>>(E, sorted_senders.p, rows, in_ptr.p);
        check_launch("sender segments");
        sender_rows = rows;
    }

    void require_edges() const {
        if (!have_edges) throw ArgError("no edge set: call smx_begin / smx_compute / smx_build_neighbors first");
    }

    // ------------------------------------------------------------------ GEMM plumbing
    void run_gemms(const std::vector<GemmProblem<T>>& list, long long max_rows, int max_cols) {
        if (list.empty() || max_rows <= 0) return;
        if (list.size() > kProblemRing) throw UnsupportedError("too many element types for one GEMM launch");
        if (ring_pos + list.size() > kProblemRing) ring_pos = 0;
        std::copy(list.begin(), list.end(), host_ring + ring_pos);
        dim3 grid(static_cast<unsigned>((max_rows + kGemmBM - 1) / kGemmBM), (max_cols + kGemmBN - 1) / kGemmBN,
                  static_cast<unsigned>(list.size()));
        if constexpr (sizeof(T) == 4) {
            if (use_tc5) {
                for (size_t q = 0; q < list.size(); ++q) host_ring[ring_pos + q].B_image = weight_image(list[q]);
                SMX_CUDA(cudaMemcpyAsync(dev_ring.p + ring_pos, host_ring + ring_pos, list.size() * sizeof(GemmProblem<T>), cudaMemcpyHostToDevice, stream));
                dim3 g5(static_cast<unsigned>((max_rows + kTc5BM - 1) / kTc5BM), (max_cols + kTc5BN - 1) / kTc5BN, static_cast<unsigned>(list.size()));
                waits_in_flight = true;
                gemm_rows_tcgen05_kernel<<<g5, kTc5Threads, kTc5SmemBytes, stream>>>(dev_ring.p + ring_pos, kernel_status.p);
                check_launch("gemm_rows_tcgen05_kernel");
                ring_pos += list.size();
                return;
            }
        }
        SMX_CUDA(cudaMemcpyAsync(dev_ring.p + ring_pos, host_ring + ring_pos, list.size() * sizeof(GemmProblem<T>), cudaMemcpyHostToDevice, stream));
        if constexpr (sizeof(T) == 8) {
            // asynchronous-copy kernel when every problem's rows, columns and leading dimension are 16-byte aligned
            bool aligned = gemm_async;
            for (const auto& q : list)
                aligned = aligned && ((q.a_node_stride | q.a_off | q.a_sub_stride | q.ldb) & 1) == 0 &&
                          (reinterpret_cast<uintptr_t>(q.A) & 15) == 0 && (reinterpret_cast<uintptr_t>(q.B) & 15) == 0;
            if (aligned) {
                gemm_rows_f64_async_kernel<<<grid, kGemmThreads, 0, stream>>>(dev_ring.p + ring_pos);
                check_launch("gemm_rows_f64_async_kernel");
                ring_pos += list.size();
                return;
            }
        }
        gemm_rows_kernel<T><<<grid, kGemmThreads, 0, stream>>>(dev_ring.p + ring_pos);
        check_launch("gemm_rows_kernel");
        ring_pos += list.size();
    }
    // Operand image of a problem's weight matrix for the tcgen05 kernel, built on first use (the weights are
    // constant after the model upload) by a small kernel on the evaluator's stream.
    const float* weight_image(const GemmProblem<float>& p) {
        const auto key = std::make_tuple(static_cast<const void*>(p.B), p.Kd, p.Nc, p.ldb, p.transB);
        auto it = weight_images.find(key);
        if (it == weight_images.end()) {
            auto buf = std::make_unique<DevBuf<float>>();
            buf->resize(tc5_image_floats(p.Kd, p.Nc), stream);
            const long long groups = static_cast<long long>(tc5_image_floats(p.Kd, p.Nc) / 8);
            const int grid = static_cast<int>(std::min<long long>((groups + 255) / 256, 4096));
            gemm_tc5_prepare_b_kernel<<<grid, 256, 0, stream>>>(p.B, p.Kd, p.Nc, p.ldb, p.transB, buf->p);
            check_launch("gemm_tc5_prepare_b_kernel");
            it = weight_images.emplace(key, std::move(buf)).first;
        }
        return it->second->p;
    }
    GemmProblem<T> problem(const T* A, T* C, const T* B, bool by_type, int type, int sub_count, long long a_ns, long long a_off,
                           long long a_ss, long long c_ns, long long c_off, long long c_ss, int Kd, int Nc, int ldb, bool transB,
                           bool acc) {
        GemmProblem<T> p{};
        p.A = A; p.C = C; p.B = B;
        p.perm = by_type ? perm.p : nullptr;
        p.seg = by_type ? type_seg.p : nullptr;
        p.seg_index = type;
        p.num_nodes = N;
        p.sub_count = sub_count;
        p.a_node_stride = a_ns; p.a_off = a_off; p.a_sub_stride = a_ss;
        p.c_node_stride = c_ns; p.c_off = c_off; p.c_sub_stride = c_ss;
        p.Kd = Kd; p.Nc = Nc; p.ldb = ldb; p.transB = transB ? 1 : 0; p.accumulate = acc ? 1 : 0;
        return p;
    }

    // ------------------------------------------------------------------ stages
    Layer0Args<T> layer0_args() {
        Layer0Args<T> a{};
        a.N = N; a.K = model.K;
        a.node_types = node_types; a.first_neigh = first_neigh.p; a.neigh_indices = neigh_indices; a.neigh_types = neigh_types;
        a.xyz = xyz; a.r = r; a.coef0 = coef0.p; a.sm = sm; a.H0_w = H0_w.p; a.order = type_order ? perm.p : nullptr;
        a.coef0_folded = fold_a0 ? coef0_folded.p : nullptr;
        // folded table: the edge sums are A0 / act on A0_adj themselves
        a.Phi0 = fold_a0 ? A0.p : Phi0.p; a.Phi0_adj = fold_a0 ? A0_adj.p : Phi0_adj.p; a.node_forces = node_forces.p;
        a.sched = work_sched.p; a.items = work_items.p; a.n_items = work_n_items.p;
        return a;
    }

    void compute_ZBL() {   // ZBL::compute_ZBL, zbl.cpp:96-125
        if (!model.has_zbl || N == 0) return;
        ZblParams z{};
        z.a_exp = model.zbl_a_exp; z.a_prefactor = model.zbl_a_prefactor; z.p = model.zbl_p;
        for (int q = 0; q < 4; ++q) z.c[q] = model.zbl_c[q];
        z.covalent_radii = zbl_radii.p; z.atomic_numbers = zbl_numbers.p;
        zbl_kernel<<<std::min((N + 127) / 128, num_sms * 8), 128, 0, stream>>>(N, node_types, first_neigh.p, neigh_types, xyz, r, z,
                                                                              node_energies.p, node_forces.p);
        check_launch("zbl_kernel");
    }
    ScalarSplines density_splines(bool first) const {
        ScalarSplines sp{};
        sp.coef = first ? A0_spl.p : A1_spl.p;
        sp.h = first ? model.A0_spline_h : model.A1_spline_h;
        sp.bins = first ? model.A0_spline_bins : model.A1_spline_bins;
        sp.num_elements = model.num_elements;
        return sp;
    }
    void compute_A_scaled(bool first) {   // MACE::compute_A0_scaled / compute_A1_scaled, mace.cpp:273-298, 681-706
        if (!(first ? model.A0_scaled : model.A1_scaled) || N == 0) return;
        DevBuf<T>& A = first ? A0 : A1;
        if (A.n != static_cast<size_t>(N) * kNumLm * model.K) throw ArgError("compute_A_scaled: A has not been computed");
        density_scale_forward_kernel<T><<<std::min(N, num_sms * 8), 128, 0, stream>>>(N, model.K, node_types, first_neigh.p, neigh_types, r,
                                                                                    density_splines(first), A.p);
        check_launch("density_scale_forward_kernel");
    }
    void reverse_A_scaled(bool first, bool zero_dxyz) {   // MACE::reverse_A0_scaled / reverse_A1_scaled, mace.cpp:300-346, 708-757
        if (!(first ? model.A0_scaled : model.A1_scaled) || N == 0) return;
        DevBuf<T>& A = first ? A0 : A1;
        DevBuf<T>& A_adj = first ? A0_adj : A1_adj;
        if (A_adj.n != static_cast<size_t>(N) * kNumLm * model.K) throw ArgError("reverse_A_scaled: the adjoint has not been computed");
        if (zero_dxyz) node_forces.zero(stream);
        density_scale_reverse_kernel<T><<<std::min(N, num_sms * 8), 128, 0, stream>>>(N, model.K, node_types, first_neigh.p, neigh_types, xyz, r,
                                                                                    density_splines(first), A.p, A_adj.p, node_forces.p);
        check_launch("density_scale_reverse_kernel");
    }

    void compute_A0() {   // MACE::compute_A0, mace.cpp:150-201
        const int K = model.K;
        if (!fold_a0) Phi0.resize(static_cast<size_t>(N) * kNumLm * K, stream);
        A0.resize(static_cast<size_t>(N) * kNumLm * K, stream);
        if (N == 0) return;
        const int block = channel_block();
        const int grid = persistent_grid(layer0_forward_kernel<T>, block, 0, N);
        layer0_forward_kernel<T><<<grid, block, 0, stream>>>(layer0_args());
        check_launch("layer0_forward_kernel");
        if (fold_a0) return;       // the table already holds H0 and the channel mix
        std::vector<GemmProblem<T>> list;
        for (int a = 0; a < model.num_elements; ++a)
            for (int l = 0; l <= kLmaxSH; ++l)
                list.push_back(problem(Phi0.p, A0.p, A0_w.p + (static_cast<size_t>(a) * (kLmaxSH + 1) + l) * K * K, true, a, 2 * l + 1,
                                       16LL * K, 1LL * l * l * K, K, 16LL * K, 1LL * l * l * K, K, K, K, K, false, false));
        run_gemms(list, 7LL * N, K);
    }

    void reverse_A0() {   // MACE::reverse_A0, mace.cpp:203-271
        const int K = model.K;
        if (A0_adj.n != static_cast<size_t>(N) * kNumLm * K) throw ArgError("reverse_A0: A0_adj has not been computed");
        if (N == 0) return;
        if (!fold_a0) {
            Phi0_adj.resize(static_cast<size_t>(N) * kNumLm * K, stream);
            std::vector<GemmProblem<T>> list;
            for (int a = 0; a < model.num_elements; ++a)
                for (int l = 0; l <= kLmaxSH; ++l)
                    list.push_back(problem(A0_adj.p, Phi0_adj.p, A0_w.p + (static_cast<size_t>(a) * (kLmaxSH + 1) + l) * K * K, true, a,
                                           2 * l + 1, 16LL * K, 1LL * l * l * K, K, 16LL * K, 1LL * l * l * K, K, K, K, K, true, false));
            run_gemms(list, 7LL * N, K);
        }
#ifndef SMX_L0R_CPT
#define SMX_L0R_CPT 2
#endif
        // SMX_L0R_CPT channels per thread; the CTA covers the same channels with fewer threads (at least one warp)
        constexpr int kCpt = SMX_L0R_CPT;
        const int block = std::max(32, ((channel_block() / kCpt + 31) / 32) * 32);
        const int grid = persistent_grid(layer0_reverse_kernel<T, kCpt>, block, 0, N);
        layer0_reverse_kernel<T, kCpt><<<grid, block, 0, stream>>>(layer0_args());
        check_launch("layer0_reverse_kernel");
    }

    // which: 0 = contraction of block 0 (M0), 1 = of the last block (M1, one output), 2 = of the middle block (Mm)
    PolyArgs<T> poly_args(int which) {
        PolyArgs<T> a{};
        a.N = N; a.K = model.K; a.node_types = node_types; a.perm = perm.p; a.type_seg = type_seg.p; a.num_types = model.num_elements;
        if (which == 2) {
            a.num_out = model.num_LM; a.num_mono = poly_fixed ? model.num_canonm : model.num_monom;
            a.prog = progm.p; a.prog_off = progm_off.p; a.prog_cnt = progm_cnt.p; a.mono_off = monom_off.p; a.coef = coefMm.p;
            a.A = Am.p; a.M = Mm.p; a.M_adj = Mm_adj.p; a.A_adj = Am_adj.p;
        } else if (which == 0) {
            a.num_out = model.num_LM; a.num_mono = poly_fixed ? model.num_canon0 : model.num_mono0;
            a.prog = prog0.p; a.prog_off = prog0_off.p; a.prog_cnt = prog0_cnt.p; a.mono_off = mono0_off.p; a.coef = coefM0.p;
            a.A = A0.p; a.M = M0.p; a.M_adj = M0_adj.p; a.A_adj = A0_adj.p;
        } else {
            a.num_out = 1; a.num_mono = poly_fixed ? model.num_canon1 : model.num_mono1;
            a.prog = prog1.p; a.prog_off = prog1_off.p; a.prog_cnt = prog1_cnt.p; a.mono_off = mono1_off.p; a.coef = coefM1.p;
            a.A = A1.p; a.M = M1.p; a.M_adj = M1_adj.p; a.A_adj = A1_adj.p;
        }
        return a;
    }
    // Nodes of one element type per thread in the straight-line contraction kernels (see PolyVec). Measured on B200:
    // forward 4 (2.2x faster than 1 in float64, 1.6x in float32), reverse 1 (2 and 3 are equal or slower: 255 registers)
#ifndef SMX_POLY_NB_FWD
#define SMX_POLY_NB_FWD 4
#endif
#ifndef SMX_POLY_NB_REV
#define SMX_POLY_NB_REV 1
#endif
    static constexpr int kPolyNodesFwd = SMX_POLY_NB_FWD, kPolyNodesRev = SMX_POLY_NB_REV;
    template <int NOUT>
    void launch_poly_fixed(int first, bool reverse) {
        const int nb = reverse ? kPolyNodesRev : kPolyNodesFwd;
        // groups of nb nodes per element type: at most one partly filled group per type
        const long long total = (static_cast<long long>(N / nb) + model.num_elements) * model.K;
        const unsigned grid = static_cast<unsigned>((total + 127) / 128);
        if (reverse) poly_fixed_reverse_kernel<T, NOUT, kPolyNodesRev><<<grid, 128, 0, stream>>>(poly_args(first));
        else poly_fixed_forward_kernel<T, NOUT, kPolyNodesFwd><<<grid, 128, 0, stream>>>(poly_args(first));
        check_launch(reverse ? "poly_fixed_reverse_kernel" : "poly_fixed_forward_kernel");
    }
    void run_poly(int first, bool reverse) {
        if (N == 0) return;
        if (poly_fixed) {
            const int nout = first != 1 ? model.num_LM : 1;
            if (nout == 1) launch_poly_fixed<1>(first, reverse);
            else if (nout == 4) launch_poly_fixed<4>(first, reverse);
            else launch_poly_fixed<9>(first, reverse);
            return;
        }
        // nodes per thread: as many as fit ~64 KB of shared memory (inputs, plus gradient accumulators in reverse)
        constexpr int NBF = sizeof(T) == 8 ? 4 : 8, NBR = sizeof(T) == 8 ? 2 : 4;
        const int block = std::min(128, ((model.K + 31) / 32) * 32);
        const int chunks = (model.K + block - 1) / block;
        if (reverse) {
            const size_t smem = 2 * static_cast<size_t>(NBR) * kNumLm * block * sizeof(T);
            SMX_CUDA(cudaFuncSetAttribute(poly_reverse_kernel<T, NBR>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
            dim3 grid((N + NBR - 1) / NBR, model.num_elements, chunks);
            poly_reverse_kernel<T, NBR><<<grid, block, smem, stream>>>(poly_args(first));
            check_launch("poly_reverse_kernel");
        } else {
            const size_t smem = static_cast<size_t>(NBF) * kNumLm * block * sizeof(T);
            SMX_CUDA(cudaFuncSetAttribute(poly_forward_kernel<T, NBF>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
            dim3 grid((N + NBF - 1) / NBF, model.num_elements, chunks);
            poly_forward_kernel<T, NBF><<<grid, block, smem, stream>>>(poly_args(first));
            check_launch("poly_forward_kernel");
        }
    }

    void compute_M0() {   // MACE::compute_M0, mace.cpp:348-370
        if (A0.n != static_cast<size_t>(N) * kNumLm * model.K) throw ArgError("compute_M0: A0 has not been computed");
        M0.resize(static_cast<size_t>(N) * model.num_LM * model.K, stream);
        run_poly(0, false);
    }
    void reverse_M0() {   // MACE::reverse_M0, mace.cpp:372-395
        if (M0_adj.n != static_cast<size_t>(N) * model.num_LM * model.K) throw ArgError("reverse_M0: M0_adj has not been computed");
        A0_adj.resize(static_cast<size_t>(N) * kNumLm * model.K, stream);
        run_poly(0, true);
    }
    void compute_M1() {   // MACE::compute_M1, mace.cpp:759-777
        if (A1.n != static_cast<size_t>(N) * kNumLm * model.K) throw ArgError("compute_M1: A1 has not been computed");
        M1.resize(static_cast<size_t>(N) * model.K, stream);
        run_poly(1, false);
    }
    void reverse_M1() {   // MACE::reverse_M1, mace.cpp:779-794
        if (M1_adj.n != static_cast<size_t>(N) * model.K) throw ArgError("reverse_M1: M1_adj has not been computed");
        A1_adj.resize(static_cast<size_t>(N) * kNumLm * model.K, stream);
        run_poly(1, true);
    }

    void compute_H1() {   // MACE::compute_H1, mace.cpp:397-423
        const int K = model.K, nLM = model.num_LM;
        if (M0.n != static_cast<size_t>(N) * nLM * K) throw ArgError("compute_H1: M0 has not been computed");
        H1.resize(static_cast<size_t>(N) * nLM * K, stream);
        h1_rows = N;
        std::vector<GemmProblem<T>> list;
        for (int l = 0; l <= model.L_max; ++l)
            list.push_back(problem(M0.p, H1.p, H1_w.p + static_cast<size_t>(l) * K * K, false, 0, 2 * l + 1, 1LL * nLM * K,
                                   1LL * l * l * K, K, 1LL * nLM * K, 1LL * l * l * K, K, K, K, K, false, false));
        run_gemms(list, static_cast<long long>(2 * model.L_max + 1) * N, K);
    }
    void reverse_H1() {   // MACE::reverse_H1, mace.cpp:425-451
        const int K = model.K, nLM = model.num_LM;
        if (H1_adj.n < static_cast<size_t>(N) * nLM * K) throw ArgError("reverse_H1: H1_adj has not been computed");
        M0_adj.resize(static_cast<size_t>(N) * nLM * K, stream);
        std::vector<GemmProblem<T>> list;
        for (int l = 0; l <= model.L_max; ++l)
            list.push_back(problem(H1_adj.p, M0_adj.p, H1_w.p + static_cast<size_t>(l) * K * K, false, 0, 2 * l + 1, 1LL * nLM * K,
                                   1LL * l * l * K, K, 1LL * nLM * K, 1LL * l * l * K, K, K, K, K, true, false));
        run_gemms(list, static_cast<long long>(2 * model.L_max + 1) * N, K);
    }

    bool deep() const { return model.num_interactions == 3; }
    // which: 1 = last block (features of the previous block: Hm in three-block models, else H1), 2 = middle block (H1)
    TPArgs<T> tp_args(int which) {
        TPArgs<T> a{};
        a.N = N; a.K = model.K;
        a.node_types = node_types; a.first_neigh = first_neigh.p; a.neigh_indices = neigh_indices; a.neigh_types = neigh_types;
        a.xyz = xyz; a.r = r; a.sm = sm;
        if (which == 2) {
            a.coef1 = coefm.p; a.H = H1.p; a.Phi1 = Phim.p; a.dPhi1 = dPhim.p; a.H_adj = H1_adj.p;
        } else {
            a.coef1 = coef1.p; a.H = deep() ? Hm.p : H1.p; a.Phi1 = Phi1.p; a.dPhi1 = dPhi1.p; a.H_adj = deep() ? Hm_adj.p : H1_adj.p;
        }
        a.Hmsg = Hmsg.p; a.node_forces = node_forces.p;
        if (radial_mlp && which == 1 && !radial_in_kernel) { a.R_edge = R_edge.p; a.Rd_edge = Rd_edge.p; }
        a.status = kernel_status.p;
        a.order = type_order ? perm.p : nullptr;
        a.sched = work_sched.p; a.items = work_items.p; a.n_items = work_n_items.p;
        return a;
    }
    template <int LF>
    void launch_tp(bool reverse, int which) {
        const int block = channel_block();
        if constexpr (sizeof(T) == 8 && LF <= 2) {     // L_max = 3 would need all 512 TMEM columns for one CTA: register kernel
            if (reverse && tmem_reverse && !staged_reverse) {
                // receiver adjoint in tensor memory: more resident CTAs (see tp_reverse_tmem_kernel). The CTAs of one SM
                // must fit into its 512 TMEM columns, or the allocation of the last one would wait for another to exit.
                constexpr int kCols = tp_tmem_cols(LF);
                // Grid: the resident CTAs per SM the kernel is compiled for (its register budget and 36 KB of shared memory
                // allow them; the occupancy query reports one CTA per SM for kernels that allocate tensor memory, although
                // several such CTAs do share an SM, so it is not used here). CTAs beyond what fits simply start later and
                // find fewer work items left.
                auto launch = [&](auto kern, int min_blocks) {
                    const int per_sm = std::max(1, std::min(min_blocks, 512 / kCols));
                    const int grid = static_cast<int>(std::max<long long>(1, std::min<long long>(static_cast<long long>(num_sms) * per_sm, N)));
                    kern<<<grid, block, 0, stream>>>(tp_args(which));
                };
                // resident CTAs per SM the kernel is compiled for (register budget 255 / 168 / 128)
                if constexpr (LF >= 2) {
                    launch(tp_reverse_tmem_kernel<LF, 2>, 2);
                } else {
                    if (tmem_min_blocks <= 2) launch(tp_reverse_tmem_kernel<LF, 2>, 2);
                    else if (tmem_min_blocks == 3) launch(tp_reverse_tmem_kernel<LF, 3>, 3);
                    else launch(tp_reverse_tmem_kernel<LF, 4>, 4);
                }
                check_launch("tp_reverse_tmem_kernel");
                return;
            }
        }
        if constexpr (sizeof(T) == 4 && LF <= 1) {
            if (reverse && radial_in_kernel) {
                // radial functions and derivatives from the un-splined network on the tensor cores inside the kernel
                constexpr int smem = RnRevSmem<LF>::kTotal;
                SMX_CUDA(cudaFuncSetAttribute(tp_reverse_rnet_kernel<LF>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
                const int grid = std::max(1, std::min(num_sms, N));
                waits_in_flight = true;
                tp_reverse_rnet_kernel<LF><<<grid, kRnThreads, smem, stream>>>(tp_args(which), rn_tiles.p, radial_source());
                check_launch("tp_reverse_rnet_kernel");
                return;
            }
        }
        if (reverse) {
            // two slots of one spline-row chunk each; staged only if that costs no resident CTA
            const size_t slots = 2 * sizeof(T) * 4 * make_tp_table(LF).P * static_cast<size_t>(std::min(model.K, block));
            bool staged = false;
            if constexpr (LF <= 2) {      // the row-staging variant is not built for L_max = 3
                staged = staged_reverse && !radial_mlp && slots <= static_cast<size_t>(max_dynamic_smem);
                int plain_per_sm = 0, staged_per_sm = 0;
                if (staged) {
                    SMX_CUDA(cudaFuncSetAttribute(tp_reverse_kernel<T, LF, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(slots)));
                    SMX_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&plain_per_sm, tp_reverse_kernel<T, LF, false>, block, 0));
                    SMX_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&staged_per_sm, tp_reverse_kernel<T, LF, true>, block, slots));
                    staged = staged_per_sm >= 1 && staged_per_sm >= plain_per_sm;
                }
                if (staged) {
                    const int grid = persistent_grid(tp_reverse_kernel<T, LF, true>, block, slots, N);
                    waits_in_flight = true;
                    tp_reverse_kernel<T, LF, true><<<grid, block, slots, stream>>>(tp_args(which));
                }
            }
            if (!staged) {
                const int grid = persistent_grid(tp_reverse_kernel<T, LF, false>, block, 0, N);
                tp_reverse_kernel<T, LF, false><<<grid, block, 0, stream>>>(tp_args(which));
            }
            check_launch("tp_reverse_kernel");
        } else {
            if constexpr (sizeof(T) == 4 && LF <= 1) {      // for L_max = 2 the 17 weight tiles exceed shared memory
                if (radial_in_kernel) {
                    // radial functions from the un-splined network on the tensor cores inside the kernel: one CTA per SM
                    constexpr int smem = RnSmem<LF>::kTotal;
                    SMX_CUDA(cudaFuncSetAttribute(tp_forward_rnet_kernel<LF>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
                    const int grid = std::max(1, std::min(num_sms, N));
                    waits_in_flight = true;
                    tp_forward_rnet_kernel<LF><<<grid, kRnThreads, smem, stream>>>(tp_args(which), rn_tiles.p, radial_source());
                    check_launch("tp_forward_rnet_kernel");
                    return;
                }
            }
            const int grid = persistent_grid(tp_forward_kernel<T, LF>, block, 0, N);
            tp_forward_kernel<T, LF><<<grid, block, 0, stream>>>(tp_args(which));
            check_launch("tp_forward_kernel");
        }
    }
    void dispatch_tp(bool reverse, int which = 1) {
        switch (model.L_max) {
            case 0: launch_tp<0>(reverse, which); break;
            case 1: launch_tp<1>(reverse, which); break;
            case 2: launch_tp<2>(reverse, which); break;
            case 3: launch_tp<3>(reverse, which); break;
            default: throw UnsupportedError("L_max > 3");
        }
    }

    // Run-time radial mode: R_edge (and Rd_edge when `with_derivative`) of the active edges from the un-splined network.
    RnHidden radial_source() const {
        RnHidden hd{};
        hd.x = rn_x.p; hd.dx = rn_dx.p; hd.basis = radial_lowrank ? rn_basis.p : nullptr; hd.sm = sm; hd.hidden = model.rmlp1.hidden;
        return hd;
    }
    void radial_hidden() {
        if (radial_lowrank) return;        // evaluated inside the fused kernels from the tabulated hidden layer
        if constexpr (sizeof(T) == 4) {
            const auto& rm = model.rmlp1;
            const int H = rm.hidden;
            if (!radial_hidden_valid) {
                rn_x.resize(static_cast<size_t>(E) * H, stream);
                rn_dx.resize(static_cast<size_t>(E) * H, stream);
                RadialNetArgs a{};
                a.N = N; a.num_bessel = rm.num_bessel; a.poly_p = rm.poly_p; a.hidden = H; a.num_hidden_layers = rm.num_hidden_layers;
                a.num_elements = model.num_elements; a.r_cut = static_cast<float>(model.r_cut); a.silu_scale = static_cast<float>(rm.silu_scale);
                a.node_types = node_types; a.first_neigh = first_neigh.p; a.neigh_types = neigh_types; a.r = r;
                a.w_first = rn_w_first.p; a.w_hidden = rn_w_hidden.p; a.pair_scale = rn_pair_scale.p; a.x_out = rn_x.p; a.dx_out = rn_dx.p;
                const size_t smem = sizeof(float) * (static_cast<size_t>(rm.num_bessel) * H + static_cast<size_t>(rm.num_hidden_layers - 1) * H * H +
                                                     kRadialGroups * 4 * 64);
                SMX_CUDA(cudaFuncSetAttribute(radial_hidden_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
                const int grid = std::max(1, std::min(N, num_sms * 4));
                radial_hidden_kernel<<<grid, kRadialGroups * 64, smem, stream>>>(a);
                check_launch("radial_hidden_kernel");
                radial_hidden_valid = true;
            }
        }
    }
    void radial_from_network(bool with_derivative) {
        if constexpr (sizeof(T) == 4) {
            const auto& rm = model.rmlp1;
            const int H = rm.hidden, F1 = model.tp.P * model.K;
            radial_hidden();
            if (E > 0x7fffffffL) throw UnsupportedError("more than 2^31 edges in one call");
            R_edge.resize(static_cast<size_t>(E) * F1, stream);
            std::vector<GemmProblem<T>> list;
            auto last_layer = [&](const float* in, T* out) {
                GemmProblem<T> p = problem(in, out, rn_w_last.p, false, 0, 1, H, 0, 0, F1, 0, 0, H, F1, F1, false, false);
                p.num_nodes = static_cast<int>(E);
                return p;
            };
            list.push_back(last_layer(rn_x.p, R_edge.p));
            if (with_derivative) {
                Rd_edge.resize(static_cast<size_t>(E) * F1, stream);
                list.push_back(last_layer(rn_dx.p, Rd_edge.p));
            }
            run_gemms(list, E, F1);
        }
    }

    // Tensor product of block `which` (1: last, 2: middle). Sender features / their adjoints: see tp_args.
    void tp_forward_stage(int which, const char* what) {   // MACE::compute_Phi1, mace.cpp:453-502
        const int K = model.K;
        const DevBuf<T>& feat = (which == 2 || !deep()) ? H1 : Hm;
        if (feat.n < static_cast<size_t>(N) * model.num_LM * K) throw ArgError(std::string(what) + ": the sender features have not been computed");
        DevBuf<T>& out = which == 2 ? Phim : Phi1;
        out.resize(static_cast<size_t>(N) * model.tp.Q * K, stream);
        if (N == 0) return;
        radial_in_kernel = false;
        if (radial_mlp && which == 1) {
            if (radial_fused && K <= 128 && model.L_max <= 1 && model.rmlp1.hidden <= kRnHidden) { radial_hidden(); radial_in_kernel = true; }
            else radial_from_network(false);
        }
        dispatch_tp(false, which);
        radial_in_kernel = false;
    }
    void tp_reverse_stage(int which, bool zero_dxyz, bool zero_adj, const char* what) {   // MACE::reverse_Phi1, mace.cpp:504-605
        const int K = model.K, nLM = model.num_LM;
        const DevBuf<T>& dphi = which == 2 ? dPhim : dPhi1;
        if (dphi.n != static_cast<size_t>(N) * model.tp.Q * K) throw ArgError(std::string(what) + ": the adjoint of the tensor product has not been computed");
        const bool to_h1 = which == 2 || !deep();
        DevBuf<T>& adj = to_h1 ? H1_adj : Hm_adj;
        const int rows = to_h1 ? h1_rows : hm_rows;
        const size_t hsize = static_cast<size_t>(rows) * nLM * K;
        if (adj.n != hsize) { adj.resize(hsize, stream, true); }
        if (zero_dxyz) node_forces.zero(stream);
        if (zero_adj) adj.zero(stream);
        if (N == 0) return;
        if (sizeof(T) == 4) {      // float32: messages are accumulated in place by the kernel
            radial_in_kernel = false;
            if (radial_mlp && which == 1) {
                if (radial_fused && K <= 128 && model.L_max <= 1 && model.rmlp1.hidden <= kRnHidden) { radial_hidden(); radial_in_kernel = true; }
                else radial_from_network(true);
            }
            dispatch_tp(true, which);
            radial_in_kernel = false;
            return;
        }
        Hmsg.resize(static_cast<size_t>(E) * nLM * K, stream);
        dispatch_tp(true, which);
        ensure_sender_lists(std::max(rows, N));
        if (E > 0) {
            const int width = nLM * K;
            const int grid = std::min(rows, num_sms * 16);
            const bool vec = sizeof(T) == 8 && width % 2 == 0 && (reinterpret_cast<uintptr_t>(Hmsg.p) & 15) == 0 &&
                             (reinterpret_cast<uintptr_t>(adj.p) & 15) == 0;
            if (vec) {
                const int block = std::min(256, ((width / 2 + 31) / 32) * 32);
                sender_gather_kernel<T, true><<<grid, block, 0, stream>>>(rows, width, in_ptr.p, in_edge.p, Hmsg.p, adj.p);
            } else {
                const int block = std::min(256, ((width + 31) / 32) * 32);
                sender_gather_kernel<T, false><<<grid, block, 0, stream>>>(rows, width, in_ptr.p, in_edge.p, Hmsg.p, adj.p);
            }
            check_launch("sender_gather_kernel");
        }
    }
    void compute_Phi1() { tp_forward_stage(1, "compute_Phi1"); }
    void reverse_Phi1(bool zero_dxyz, bool zero_H1_adj) { tp_reverse_stage(1, zero_dxyz, zero_H1_adj, "reverse_Phi1"); }

    void linear_A_forward(int which, const char* what) {   // MACE::compute_A1, mace.cpp:607-642
        const int K = model.K;
        const TPTable& tp = model.tp;
        DevBuf<T>& phi = which == 2 ? Phim : Phi1;
        DevBuf<T>& out = which == 2 ? Am : A1;
        const T* w = which == 2 ? Am_w.p : A1_w.p;
        const auto& off = which == 2 ? model.Am_w_off : model.A1_w_off;
        if (phi.n != static_cast<size_t>(N) * tp.Q * K) throw ArgError(std::string(what) + ": the tensor product has not been computed");
        out.resize(static_cast<size_t>(N) * kNumLm * K, stream);
        std::vector<GemmProblem<T>> list;
        for (int l = 0; l <= kLmaxSH; ++l)
            list.push_back(problem(phi.p, out.p, w + off[l], false, 0, 2 * l + 1, 1LL * tp.Q * K, 1LL * tp.lme_off[l] * K,
                                   1LL * tp.n_e[l] * K, 16LL * K, 1LL * l * l * K, K, tp.n_e[l] * K, K, K, false, false));
        run_gemms(list, 7LL * N, K);
    }
    void linear_A_reverse(int which, const char* what) {   // MACE::reverse_A1, mace.cpp:644-679
        const int K = model.K;
        const TPTable& tp = model.tp;
        DevBuf<T>& adj = which == 2 ? Am_adj : A1_adj;
        DevBuf<T>& dphi = which == 2 ? dPhim : dPhi1;
        const T* w = which == 2 ? Am_w.p : A1_w.p;
        const auto& off = which == 2 ? model.Am_w_off : model.A1_w_off;
        if (adj.n != static_cast<size_t>(N) * kNumLm * K) throw ArgError(std::string(what) + ": the adjoint of A has not been computed");
        dphi.resize(static_cast<size_t>(N) * tp.Q * K, stream);
        std::vector<GemmProblem<T>> list;
        int max_cols = K;
        for (int l = 0; l <= kLmaxSH; ++l) {
            list.push_back(problem(adj.p, dphi.p, w + off[l], false, 0, 2 * l + 1, 16LL * K, 1LL * l * l * K, K,
                                   1LL * tp.Q * K, 1LL * tp.lme_off[l] * K, 1LL * tp.n_e[l] * K, K, tp.n_e[l] * K, K, true, false));
            max_cols = std::max(max_cols, tp.n_e[l] * K);
        }
        run_gemms(list, 7LL * N, max_cols);
    }
    void compute_A1() { linear_A_forward(1, "compute_A1"); }
    void reverse_A1() { linear_A_reverse(1, "reverse_A1"); }

    // ---- middle interaction block (three-block models): Phim -> Am -> Mm -> Hm, the generalisation of the last block's
    // stages to a contraction with every (L, M) (as compute_M0) and features Hm = Mm . W_L + H1 . W_res[type][L]
    void require_deep(const char* what) const {
        if (!deep()) throw ArgError(std::string(what) + ": the model has two interaction blocks");
    }
    void compute_Phim() { require_deep("compute_Phim"); tp_forward_stage(2, "compute_Phim"); }
    void compute_Am() { require_deep("compute_Am"); linear_A_forward(2, "compute_Am"); }
    void compute_Mm() {
        require_deep("compute_Mm");
        if (Am.n != static_cast<size_t>(N) * kNumLm * model.K) throw ArgError("compute_Mm: Am has not been computed");
        Mm.resize(static_cast<size_t>(N) * model.num_LM * model.K, stream);
        run_poly(2, false);
    }
    void compute_Hm() {
        require_deep("compute_Hm");
        const int K = model.K, nLM = model.num_LM;
        if (Mm.n != static_cast<size_t>(N) * nLM * K) throw ArgError("compute_Hm: Mm has not been computed");
        Hm.resize(static_cast<size_t>(N) * nLM * K, stream);
        hm_rows = N;
        std::vector<GemmProblem<T>> list;
        for (int l = 0; l <= model.L_max; ++l)
            list.push_back(problem(Mm.p, Hm.p, Hm_w.p + static_cast<size_t>(l) * K * K, false, 0, 2 * l + 1, 1LL * nLM * K,
                                   1LL * l * l * K, K, 1LL * nLM * K, 1LL * l * l * K, K, K, K, K, false, false));
        run_gemms(list, static_cast<long long>(2 * model.L_max + 1) * N, K);
        list.clear();
        for (int a = 0; a < model.num_elements; ++a)
            for (int l = 0; l <= model.L_max; ++l)
                list.push_back(problem(H1.p, Hm.p, Hm_res.p + (static_cast<size_t>(a) * (model.L_max + 1) + l) * K * K, true, a, 2 * l + 1,
                                       1LL * nLM * K, 1LL * l * l * K, K, 1LL * nLM * K, 1LL * l * l * K, K, K, K, K, false, true));
        run_gemms(list, static_cast<long long>(2 * model.L_max + 1) * N, K);
    }
    void reverse_Hm() {
        require_deep("reverse_Hm");
        const int K = model.K, nLM = model.num_LM;
        if (Hm_adj.n < static_cast<size_t>(N) * nLM * K) throw ArgError("reverse_Hm: Hm_adj has not been computed");
        if (H1_adj.n < static_cast<size_t>(N) * nLM * K) throw ArgError("reverse_Hm: H1_adj has not been computed");
        Mm_adj.resize(static_cast<size_t>(N) * nLM * K, stream);
        std::vector<GemmProblem<T>> list;
        for (int l = 0; l <= model.L_max; ++l)
            list.push_back(problem(Hm_adj.p, Mm_adj.p, Hm_w.p + static_cast<size_t>(l) * K * K, false, 0, 2 * l + 1, 1LL * nLM * K,
                                   1LL * l * l * K, K, 1LL * nLM * K, 1LL * l * l * K, K, K, K, K, true, false));
        for (int a = 0; a < model.num_elements; ++a)
            for (int l = 0; l <= model.L_max; ++l)
                list.push_back(problem(Hm_adj.p, H1_adj.p, Hm_res.p + (static_cast<size_t>(a) * (model.L_max + 1) + l) * K * K, true, a,
                                       2 * l + 1, 1LL * nLM * K, 1LL * l * l * K, K, 1LL * nLM * K, 1LL * l * l * K, K, K, K, K, true, true));
        run_gemms(list, static_cast<long long>(2 * model.L_max + 1) * N, K);
    }
    void reverse_Mm() {
        require_deep("reverse_Mm");
        if (Mm_adj.n != static_cast<size_t>(N) * model.num_LM * model.K) throw ArgError("reverse_Mm: Mm_adj has not been computed");
        Am_adj.resize(static_cast<size_t>(N) * kNumLm * model.K, stream);
        run_poly(2, true);
    }
    void reverse_Am() { require_deep("reverse_Am"); linear_A_reverse(2, "reverse_Am"); }
    void reverse_Phim(bool zero_dxyz, bool zero_H1_adj) { require_deep("reverse_Phim"); tp_reverse_stage(2, zero_dxyz, zero_H1_adj, "reverse_Phim"); }

    void compute_H2() {   // MACE::compute_H2, mace.cpp:796-832
        const int K = model.K, nLM = model.num_LM;
        if (M1.n != static_cast<size_t>(N) * K) throw ArgError("compute_H2: M1 has not been computed");
        H2.resize(static_cast<size_t>(N) * K, stream);
        std::vector<GemmProblem<T>> list;
        for (int a = 0; a < model.num_elements; ++a)
            list.push_back(problem(deep() ? Hm.p : H1.p, H2.p, H2_w_H1.p + static_cast<size_t>(a) * K * K, true, a, 1, 1LL * nLM * K, 0, 0, K, 0, 0, K, K, K,
                                   false, false));   // residual of the previous block's scalar features
        run_gemms(list, N, K);
        list.clear();
        list.push_back(problem(M1.p, H2.p, H2_w_M1.p, false, 0, 1, K, 0, 0, K, 0, 0, K, K, K, false, true));
        run_gemms(list, N, K);
    }
    void reverse_H2(bool zero_H1_adj) {   // MACE::reverse_H2, mace.cpp:834-874
        const int K = model.K, nLM = model.num_LM;
        if (H2_adj.n != static_cast<size_t>(N) * K) throw ArgError("reverse_H2: H2_adj has not been computed");
        DevBuf<T>& prev_adj = deep() ? Hm_adj : H1_adj;
        const size_t hsize = static_cast<size_t>(deep() ? hm_rows : h1_rows) * nLM * K;
        if (prev_adj.n != hsize) prev_adj.resize(hsize, stream, true);
        M1_adj.resize(static_cast<size_t>(N) * K, stream);
        if (zero_H1_adj) prev_adj.zero(stream);
        std::vector<GemmProblem<T>> list;
        for (int a = 0; a < model.num_elements; ++a)
            list.push_back(problem(H2_adj.p, prev_adj.p, H2_w_H1.p + static_cast<size_t>(a) * K * K, true, a, 1, K, 0, 0, 1LL * nLM * K, 0, 0, K, K,
                                   K, true, true));
        list.push_back(problem(H2_adj.p, M1_adj.p, H2_w_M1.p, false, 0, 1, K, 0, 0, K, 0, 0, K, K, K, true, false));
        run_gemms(list, N, K);
    }

    void compute_readouts() {   // MACE::compute_readouts, mace.cpp:876-903
        const int K = model.K, nLM = model.num_LM;
        if (H2.n != static_cast<size_t>(N) * K) throw ArgError("compute_readouts: H2 has not been computed");
        H1_adj.resize(static_cast<size_t>(h1_rows) * nLM * K, stream);
        H1_adj.zero(stream);
        H2_adj.resize(static_cast<size_t>(N) * K, stream);
        if (deep()) {
            Hm_adj.resize(static_cast<size_t>(hm_rows) * nLM * K, stream);
            Hm_adj.zero(stream);
        }
        if (N == 0) return;
        ReadoutArgs<T> a{};
        a.N = N; a.K = K; a.nLM = nLM; a.node_types = node_types; a.E0 = E0.p;
        a.ro1 = ro1.p; a.W1 = ro2_w1.p; a.w2 = ro2_w2.p; a.scale = static_cast<T>(model.ro2_scale);
        a.H1 = H1.p; a.H2 = H2.p; a.node_energies = node_energies.p; a.H1_adj = H1_adj.p; a.H2_adj = H2_adj.p;
        if (deep()) { a.ro_m = ro_m.p; a.Hm = Hm.p; a.Hm_adj = Hm_adj.p; }
        const int block = 128;
        const int grid = std::min((N + 3) / 4, num_sms * 16);
        readout_kernel<T><<<grid, block, 0, stream>>>(a);
        check_launch("readout_kernel");
    }

    void stage(const std::string& s, bool zero_dxyz, bool zero_H1_adj) override {
        require_edges();
        SMX_CUDA(cudaSetDevice(device));
        NvtxRange range(s.c_str());
        if (s == "compute_Y" || s == "compute_R0" || s == "compute_R1") return;  // fused into the edge kernels
        if (s == "compute_A0") compute_A0();
        else if (s == "compute_ZBL") compute_ZBL();
        else if (s == "compute_A0_scaled") compute_A_scaled(true);
        else if (s == "compute_A1_scaled") compute_A_scaled(false);
        else if (s == "reverse_A0_scaled") reverse_A_scaled(true, false);
        else if (s == "reverse_A1_scaled") reverse_A_scaled(false, zero_dxyz);
        else if (s == "compute_M0") compute_M0();
        else if (s == "compute_H1") compute_H1();
        else if (s == "compute_Phi1") compute_Phi1();
        else if (s == "compute_A1") compute_A1();
        else if (s == "compute_M1") compute_M1();
        else if (s == "compute_H2") compute_H2();
        else if (s == "compute_readouts") compute_readouts();
        else if (s == "reverse_H2") reverse_H2(zero_H1_adj);
        else if (s == "reverse_M1") reverse_M1();
        else if (s == "reverse_A1") reverse_A1();
        else if (s == "reverse_Phi1") reverse_Phi1(zero_dxyz, zero_H1_adj);
        else if (s == "reverse_H1") reverse_H1();
        else if (s == "reverse_M0") reverse_M0();
        else if (s == "reverse_A0") reverse_A0();
        else if (s == "compute_Rm") return;   // fused, like compute_R1
        else if (s == "compute_Phim") compute_Phim();
        else if (s == "compute_Am") compute_Am();
        else if (s == "compute_Mm") compute_Mm();
        else if (s == "compute_Hm") compute_Hm();
        else if (s == "reverse_Hm") reverse_Hm();
        else if (s == "reverse_Mm") reverse_Mm();
        else if (s == "reverse_Am") reverse_Am();
        else if (s == "reverse_Phim") reverse_Phim(zero_dxyz, zero_H1_adj);
        else throw ArgError("unknown stage '" + s + "'");
    }

    void sync() override {
        SMX_CUDA(cudaSetDevice(device));
        check_kernel_status();
    }
    // Issue all further work on the caller's stream (`external`), or go back to the evaluator's own stream.
    // A null handle with `external` set means the legacy default stream.
    void set_stream(void* s, bool external) override {
        SMX_CUDA(cudaSetDevice(device));
        SMX_CUDA(cudaStreamSynchronize(stream));
        if (external) {
            if (own_stream) own_stream_handle = stream;
            stream = static_cast<cudaStream_t>(s);
            own_stream = false;
        } else if (!own_stream) {
            stream = own_stream_handle;
            own_stream = true;
        }
    }
    // Keep only the first `num_nodes` receivers of the current edge set (their rows are a prefix of the edge arrays).
    // Make the first `num_nodes` receivers of the edge set the active ones. Without `keep_outputs` this starts a new
    // evaluation (outputs zero-filled); with it the evaluation in progress continues on the other receiver set.
    long restrict_nodes(int num_nodes, bool keep_outputs) override {
        require_edges();
        SMX_CUDA(cudaSetDevice(device));
        if (num_nodes < 0 || num_nodes > N_built) throw ArgError("restrict_nodes: num_nodes out of range");
        // The row offsets of an edge set are read back once (the only host synchronisation, at the first call after the
        // edge set changed); every later switch of the receiver set is a host-side lookup.
        if (!first_host_valid) {
            first_host.resize(static_cast<size_t>(N_built) + 1);
            SMX_CUDA(cudaMemcpyAsync(first_host.data(), first_neigh.p, first_host.size() * sizeof(long long), cudaMemcpyDeviceToHost, stream));
            SMX_CUDA(cudaStreamSynchronize(stream));
            first_host_valid = true;
        }
        const long long e = first_host[num_nodes];
        adopt_edges(num_nodes, static_cast<long>(e), keep_outputs, false);
        return static_cast<long>(e);
    }
    // Grow H1 / H1_adj to `rows` feature rows keeping the existing rows (ghost rows are appended by the caller).
    void resize_rows(const std::string& name, int rows) override {
        SMX_CUDA(cudaSetDevice(device));
        if (name != "H1" && name != "H1_adj" && name != "Hm" && name != "Hm_adj")
            throw ArgError("resize_rows: only H1, Hm and their adjoints have ghost rows");
        if (rows < N) throw ArgError("resize_rows: fewer rows than nodes");
        DevBuf<T>& b = name == "H1" ? H1 : name == "H1_adj" ? H1_adj : name == "Hm" ? Hm : Hm_adj;
        const size_t old = b.n, want = static_cast<size_t>(rows) * model.num_LM * model.K;
        b.resize(want, stream, true);
        if (want > old) SMX_CUDA(cudaMemsetAsync(b.p + old, 0, (want - old) * sizeof(T), stream));
        if (name == "H1") h1_rows = rows;
        if (name == "Hm") hm_rows = rows;
    }
    void* device_ptr(const std::string& name, long* count, int* elem_bytes) override {
        if (name == "atom_forces") {
            if (count) *count = static_cast<long>(atom_f.n);
            if (elem_bytes) *elem_bytes = 8;
            return atom_f.p;
        }
        Field f = field(name);
        if (count) *count = static_cast<long>(f.t ? f.t->n : f.d->n);
        if (elem_bytes) *elem_bytes = f.t ? static_cast<int>(sizeof(T)) : 8;
        return f.t ? static_cast<void*>(f.t->p) : static_cast<void*>(f.d->p);
    }
    // Test switch: make the first weight-tile wait of every tcgen05 GEMM CTA run out after `polls` polls (0: normal operation).
    void expire_waits(int polls) override {
        SMX_CUDA(cudaSetDevice(device));
        if (polls < 0) throw ArgError("expire_waits: negative poll count");
        SMX_CUDA(cudaMemcpyAsync(kernel_status.p + 1, &polls, sizeof(int), cudaMemcpyHostToDevice, stream));
        SMX_CUDA(cudaStreamSynchronize(stream));
    }
    // Synchronises the stream and reports a kernel whose bounded mbarrier wait ran out.
    void check_kernel_status() {
        int code = 0;
        if (waits_in_flight) SMX_CUDA(cudaMemcpyAsync(&code, kernel_status.p, sizeof(int), cudaMemcpyDeviceToHost, stream));
        SMX_CUDA(cudaStreamSynchronize(stream));
        waits_in_flight = false;
        if (code != 0) {
            // re-arm the status word: later evaluations on this handle are judged on their own kernels
            SMX_CUDA(cudaMemsetAsync(kernel_status.p, 0, sizeof(int), stream));
            SMX_CUDA(cudaStreamSynchronize(stream));
        }
        if (code != 0) throw CudaError("a bounded mbarrier wait ran out in a device kernel (code " + std::to_string(code) + "); results are invalid");
    }
    // Duration of one pass of row_stream_probe_kernel over the current edge set (best of three after a warm-up)
    // and the bytes it moves from the spline table of interaction layer `layer`.
    void measure_row_stream(int layer, double* ms, double* bytes) override {
        require_edges();
        if (layer != 0 && layer != 1) throw ArgError("measure_row_stream: layer must be 0 or 1");
        SMX_CUDA(cudaSetDevice(device));
        const int K = model.K, P = layer == 0 ? kLmaxSH + 1 : model.tp.P;
        const T* table = layer == 0 ? coef0.p : coef1.p;
        DevBuf<T> sink;
        sink.resize(1, stream);
        const int block = channel_block();
        const int grid = persistent_grid(row_stream_probe_kernel<T>, block, 0, N);
        float best = 0.f;
        for (int rep = 0; rep < 4; ++rep) {
            SMX_CUDA(cudaEventRecord(evt0, stream));
            row_stream_probe_kernel<T><<<grid, block, 0, stream>>>(N, K, P, node_types, first_neigh.p, neigh_types, r, table, sm,
                                                                    type_order ? perm.p : nullptr, sink.p);
            check_launch("row_stream_probe_kernel");
            SMX_CUDA(cudaEventRecord(evt1, stream));
            SMX_CUDA(cudaEventSynchronize(evt1));
            float t = 0.f;
            SMX_CUDA(cudaEventElapsedTime(&t, evt0, evt1));
            if (rep > 0 && (best == 0.f || t < best)) best = t;
        }
        if (ms) *ms = best;
        if (bytes) *bytes = static_cast<double>(E) * 4.0 * P * K * sizeof(T);
    }
    // Counts the entries of the current edge set that are out of range or inconsistent (see validate_inputs_kernel);
    // returns their total. `feature_rows` is the row count the sender indices may address (>= the receiver count).
    long validate_inputs(int feature_rows, long* counts) override {
        require_edges();
        SMX_CUDA(cudaSetDevice(device));
        if (feature_rows < N) throw ArgError("validate_inputs: feature_rows is smaller than the number of receivers");
        DevBuf<unsigned long long> bad;
        bad.resize(kNumInputChecks, stream);
        bad.zero(stream);
        const long long work = std::max<long long>(E, N);
        const int grid = static_cast<int>(std::min<long long>(std::max<long long>((work + 255) / 256, 1), num_sms * 16LL));
        validate_inputs_kernel<<<grid, 256, 0, stream>>>(N, E, model.num_elements, feature_rows, model.r_cut, node_types, num_neigh,
                                                       first_neigh.p, neigh_indices, neigh_types, xyz, r, bad.p);
        check_launch("validate_inputs_kernel");
        unsigned long long host[kNumInputChecks] = {};
        SMX_CUDA(cudaMemcpyAsync(host, bad.p, sizeof(host), cudaMemcpyDeviceToHost, stream));
        SMX_CUDA(cudaStreamSynchronize(stream));
        long total = 0;
        for (int c = 0; c < kNumInputChecks; ++c) {
            if (counts) counts[c] = static_cast<long>(host[c]);
            total += static_cast<long>(host[c]);
        }
        return total;
    }
    void timer_start() override {
        SMX_CUDA(cudaSetDevice(device));
        SMX_CUDA(cudaEventRecord(evt0, stream));
    }
    double timer_stop() override {
        SMX_CUDA(cudaSetDevice(device));
        SMX_CUDA(cudaEventRecord(evt1, stream));
        SMX_CUDA(cudaEventSynchronize(evt1));
        float ms = 0.f;
        SMX_CUDA(cudaEventElapsedTime(&ms, evt0, evt1));
        return ms;
    }

    void compute_all() override {   // order of MACE::compute_node_energies_forces, mace.cpp:17-64
        require_edges();
        SMX_CUDA(cudaSetDevice(device));
        static const char* names2[] = {"compute_A0", "compute_M0", "compute_H1", "compute_Phi1", "compute_A1", "compute_M1",
                                       "compute_H2", "compute_readouts", "reverse_H2", "reverse_M1", "reverse_A1", "reverse_Phi1",
                                       "reverse_H1", "reverse_M0", "reverse_A0"};
        static const char* names3[] = {"compute_A0", "compute_M0", "compute_H1", "compute_Phim", "compute_Am", "compute_Mm", "compute_Hm",
                                       "compute_Phi1", "compute_A1", "compute_M1", "compute_H2", "compute_readouts", "reverse_H2",
                                       "reverse_M1", "reverse_A1", "reverse_Phi1", "reverse_Hm", "reverse_Mm", "reverse_Am", "reverse_Phim",
                                       "reverse_H1", "reverse_M0", "reverse_A0"};
        const char* const* names = deep() ? names3 : names2;
        const int kStages = deep() ? 23 : 15;
        if (profiling && static_cast<int>(stage_events.size()) < kStages + 1) {
            while (static_cast<int>(stage_events.size()) < kStages + 1) {
                cudaEvent_t e;
                SMX_CUDA(cudaEventCreate(&e));
                stage_events.push_back(e);
            }
        }
        int mark = 0;
        NvtxRange whole("smx_compute");
        struct StageRange { bool open = false; ~StageRange() { if (open) nvtxRangePop(); } } stage_range;
        // one NVTX range per stage, closed when the next stage starts (or when an exception leaves this function)
        auto tick = [&]() {
            if (stage_range.open) nvtxRangePop();
            stage_range.open = mark < kStages;
            if (stage_range.open) nvtxRangePushA(names[mark]);
            if (profiling) SMX_CUDA(cudaEventRecord(stage_events[mark], stream));
            ++mark;
        };
        SMX_CUDA(cudaEventRecord(ev0, stream));
        compute_ZBL();
        tick(); compute_A0(); compute_A_scaled(true); tick(); compute_M0(); tick(); compute_H1();
        if (deep()) { tick(); compute_Phim(); tick(); compute_Am(); tick(); compute_Mm(); tick(); compute_Hm(); }
        tick(); compute_Phi1(); tick(); compute_A1(); compute_A_scaled(false); tick(); compute_M1(); tick(); compute_H2();
        tick(); compute_readouts();
        tick(); reverse_H2(false); tick(); reverse_M1(); reverse_A_scaled(false, false); tick(); reverse_A1(); tick(); reverse_Phi1(false, false);
        if (deep()) { tick(); reverse_Hm(); tick(); reverse_Mm(); tick(); reverse_Am(); tick(); reverse_Phim(false, false); }
        tick(); reverse_H1(); tick(); reverse_M0(); reverse_A_scaled(true, false); tick(); reverse_A0(); tick();
        SMX_CUDA(cudaEventRecord(ev1, stream));
        check_kernel_status();
        float ms = 0.f;
        SMX_CUDA(cudaEventElapsedTime(&ms, ev0, ev1));
        last_ms = ms;
        if (profiling) {
            stage_ms.clear();
            for (int sidx = 0; sidx < kStages; ++sidx) {
                float t = 0.f;
                SMX_CUDA(cudaEventElapsedTime(&t, stage_events[sidx], stage_events[sidx + 1]));
                stage_ms.emplace_back(names[sidx], t);
            }
        }
    }

    // ------------------------------------------------------------------ array access
    struct Field { DevBuf<T>* t = nullptr; DevBuf<double>* d = nullptr; };
    Field field(const std::string& s) {
        Field f;
        if (s == "node_energies") f.d = &node_energies;
        else if (s == "node_forces") f.d = &node_forces;
        else if (s == "A0") f.t = &A0;
        else if (s == "A0_adj") f.t = &A0_adj;
        else if (s == "M0") f.t = &M0;
        else if (s == "M0_adj") f.t = &M0_adj;
        else if (s == "H1") f.t = &H1;
        else if (s == "H1_adj") f.t = &H1_adj;
        else if (s == "Phi1") f.t = &Phi1;
        else if (s == "Phi1_adj") f.t = &dPhi1;
        else if (s == "A1") f.t = &A1;
        else if (s == "A1_adj") f.t = &A1_adj;
        else if (s == "M1") f.t = &M1;
        else if (s == "M1_adj") f.t = &M1_adj;
        else if (s == "H2") f.t = &H2;
        else if (s == "H2_adj") f.t = &H2_adj;
        else if (s == "Phim") f.t = &Phim;
        else if (s == "Phim_adj") f.t = &dPhim;
        else if (s == "Am") f.t = &Am;
        else if (s == "Am_adj") f.t = &Am_adj;
        else if (s == "Mm") f.t = &Mm;
        else if (s == "Mm_adj") f.t = &Mm_adj;
        else if (s == "Hm") f.t = &Hm;
        else if (s == "Hm_adj") f.t = &Hm_adj;
        else throw ArgError("unknown array '" + s + "'");
        return f;
    }

    long get_array(const std::string& name, double* dst, long cap, int mem_space) override {
        SMX_CUDA(cudaSetDevice(device));
        Field f = field(name);
        const size_t n = f.t ? f.t->n : f.d->n;
        const size_t ncopy = std::min<size_t>(n, cap < 0 ? 0 : static_cast<size_t>(cap));
        if (ncopy == 0 || !dst) return static_cast<long>(n);
        const double* src = nullptr;
        if (f.t) {
            scratch_d.resize(ncopy, stream);
            convert_kernel<T, double><<<static_cast<int>(std::min<size_t>((ncopy + 255) / 256, 4096)), 256, 0, stream>>>(
                static_cast<long long>(ncopy), f.t->p, scratch_d.p);
            check_launch("convert_kernel");
            src = scratch_d.p;
        } else {
            src = f.d->p;
        }
        SMX_CUDA(cudaMemcpyAsync(dst, src, ncopy * sizeof(double),
                                 mem_space == SMX_DEVICE ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost, stream));
        check_kernel_status();
        return static_cast<long>(n);
    }

    void set_array(const std::string& name, const double* src, long n, int mem_space) override {
        SMX_CUDA(cudaSetDevice(device));
        if (n < 0 || (n > 0 && !src)) throw ArgError("set_array: bad source");
        Field f = field(name);
        if (f.d) {
            f.d->resize(n, stream);
            if (n) SMX_CUDA(cudaMemcpyAsync(f.d->p, src, n * sizeof(double),
                                           mem_space == SMX_DEVICE ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, stream));
        } else {
            f.t->resize(n, stream);
            const double* dsrc = src;
            if (mem_space != SMX_DEVICE) {
                scratch_d.resize(n, stream);
                if (n) SMX_CUDA(cudaMemcpyAsync(scratch_d.p, src, n * sizeof(double), cudaMemcpyHostToDevice, stream));
                dsrc = scratch_d.p;
            }
            if (n) {
                convert_kernel<double, T><<<static_cast<int>(std::min<size_t>((n + 255) / 256, 4096)), 256, 0, stream>>>(n, dsrc, f.t->p);
                check_launch("convert_kernel");
            }
        }
        if (name == "H1" || name == "H1_adj" || name == "Hm" || name == "Hm_adj") {
            const size_t row = static_cast<size_t>(model.num_LM) * model.K;
            if (static_cast<size_t>(n) % row != 0) throw ArgError("set_array: feature array length is not a multiple of num_LM * num_channels");
            const int rows = static_cast<int>(static_cast<size_t>(n) / row);
            if (name == "H1") h1_rows = rows;
            if (name == "Hm") hm_rows = rows;
        }
        SMX_CUDA(cudaStreamSynchronize(stream));
    }

    // Per-atom forces of the current edge set into the device array "atom_forces" (at least `rows` rows of 3), asynchronous.
    void atom_forces(int rows) override {
        require_edges();
        SMX_CUDA(cudaSetDevice(device));
        if (rows < N) throw ArgError("atom_forces: num_rows must be at least num_nodes");
        ensure_sender_lists(std::max(rows, std::max(h1_rows, N)));
        const int srows = sender_rows;
        atom_f.resize(3 * static_cast<size_t>(srows), stream);
        if (srows > 0) {
            atom_forces_kernel<<<std::min((srows + 3) / 4, num_sms * 16), 128, 0, stream>>>(srows, N, first_neigh.p, in_ptr.p, in_edge.p,
                                                                                              node_forces.p, atom_f.p);
            check_launch("atom_forces_kernel");
        }
    }

    // ------------------------------------------------------------------ halo rows (see rows_gather_kernel)
    // Row width and storage of a named array that has halo rows: the feature arrays (num_LM * K values of T) and the
    // per-atom forces (3 doubles).
    template <typename F>
    void with_halo_array(const std::string& name, F&& fn) {
        if (name == "atom_forces") { fn(atom_f.p, atom_f.n, 3); return; }
        if (name != "H1" && name != "H1_adj" && name != "Hm" && name != "Hm_adj")
            throw ArgError("halo: only H1, Hm, their adjoints and atom_forces have halo rows");
        Field f = field(name);
        fn(f.t->p, f.t->n, model.num_LM * model.K);
    }
    static int copy_grid(long long total, int num_sms) { return static_cast<int>(std::min<long long>((total + 255) / 256, num_sms * 32LL)); }
    void halo_pack(const std::string& name, const int* rows, int n, void* dst) override {
        SMX_CUDA(cudaSetDevice(device));
        if (n < 0 || (n > 0 && (!rows || !dst))) throw ArgError("halo_pack: bad arguments");
        if (n == 0) return;
        with_halo_array(name, [&](auto* p, size_t, int width) {
            using U = std::remove_pointer_t<decltype(p)>;
            const long long total = static_cast<long long>(n) * width;
            rows_gather_kernel<U><<<copy_grid(total, num_sms), 256, 0, stream>>>(p, width, rows, total, static_cast<U*>(dst));
        });
        check_launch("rows_gather_kernel");
    }
    void halo_unpack(const std::string& name, const int* rows, int n, const void* src, bool add) override {
        SMX_CUDA(cudaSetDevice(device));
        if (n < 0 || (n > 0 && (!rows || !src))) throw ArgError("halo_unpack: bad arguments");
        if (n == 0) return;
        const int* grouped_rows = nullptr;
        const int* grouped_pos = nullptr;
        if (add) {
            // group the list positions by destination row (stable), so each row is summed by one thread in list order
            DevBuf<int>* out_rows = &halo_rows;
            DevBuf<int>* out_pos = &halo_pos;
            bool have = false;
            if (halo_cache) {
                auto [it, fresh] = halo_groupings.try_emplace({rows, n});
                if (fresh) { it->second.rows = std::make_unique<DevBuf<int>>(); it->second.pos = std::make_unique<DevBuf<int>>(); }
                out_rows = it->second.rows.get(); out_pos = it->second.pos.get();
                have = !fresh;
            }
            if (!have) {
                halo_iota.resize(n, stream); out_rows->resize(n, stream); out_pos->resize(n, stream);
                iota_kernel<<<std::min(1024, (n + 255) / 256), 256, 0, stream>>>(n, halo_iota.p);
                check_launch("iota");
                size_t bytes = 0;
                SMX_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, bytes, rows, out_rows->p, halo_iota.p, out_pos->p, n, 0, 32, stream));
                cub_tmp.resize(bytes, stream);
                SMX_CUDA(cub::DeviceRadixSort::SortPairs(cub_tmp.p, bytes, rows, out_rows->p, halo_iota.p, out_pos->p, n, 0, 32, stream));
                launches += 1;
            }
            grouped_rows = out_rows->p; grouped_pos = out_pos->p;
        }
        with_halo_array(name, [&](auto* p, size_t, int width) {
            using U = std::remove_pointer_t<decltype(p)>;
            const long long total = static_cast<long long>(n) * width;
            if (add) rows_scatter_add_kernel<U><<<copy_grid(total, num_sms), 256, 0, stream>>>(p, width, grouped_rows, grouped_pos, n, static_cast<const U*>(src));
            else rows_scatter_kernel<U><<<copy_grid(total, num_sms), 256, 0, stream>>>(p, width, rows, total, static_cast<const U*>(src));
        });
        check_launch(add ? "rows_scatter_add_kernel" : "rows_scatter_kernel");
    }
    // Keep (enable != 0) or drop and stop keeping (0) the groupings of unpack-add index lists. A kept grouping is reused whenever
    // a list of the same address and length comes again, so it is for callers whose lists do not change in place.
    void halo_cache_lists(int enable) override {
        SMX_CUDA(cudaSetDevice(device));
        if (!enable) {
            SMX_CUDA(cudaStreamSynchronize(stream));      // a kernel may still read a grouping about to be freed
            halo_groupings.clear();
        }
        halo_cache = enable != 0;
    }
    // ------------------------------------------------------------------ halo exchange over NCCL (see nccl_transport.hpp)
    NcclApi::Comm comm = nullptr;
    int comm_rank = -1, comm_size = 0;
    std::vector<std::unique_ptr<DevBuf<unsigned char>>> xbuf_send, xbuf_recv;
    DevBuf<double> reduce_buf;
    void comm_init(const void* id, int id_bytes, int nranks, int rank) override {
        SMX_CUDA(cudaSetDevice(device));
        if (id_bytes != static_cast<int>(sizeof(NcclApi::UniqueId)) || !id || nranks < 1 || rank < 0 || rank >= nranks)
            throw ArgError("comm_init: bad arguments (the id is the 128 bytes of smx_comm_unique_id)");
        const NcclApi& nccl = NcclApi::get();
        comm_destroy();
        NcclApi::UniqueId uid;
        std::memcpy(&uid, id, sizeof(uid));
        nccl.check(nccl.CommInitRank(&comm, nranks, uid, rank), "ncclCommInitRank");
        comm_rank = rank; comm_size = nranks;
    }
    void comm_destroy() override {
        if (comm) { NcclApi::get().CommDestroy(comm); comm = nullptr; comm_rank = -1; comm_size = 0; }
    }
    // One exchange with `num_peers` slab neighbours on the evaluator's stream: pack the rows send_rows[q] of `name`, grouped
    // ncclSend / ncclRecv, unpack into the rows recv_rows[q] (copy, or fixed-order add). No host synchronisation.
    void halo_exchange(const std::string& name, bool add, int num_peers, const int* peers, const int* const* send_rows,
                       const int* send_counts, const int* const* recv_rows, const int* recv_counts) override {
        SMX_CUDA(cudaSetDevice(device));
        if (!comm) throw ArgError("halo_exchange: call smx_comm_init first");
        if (num_peers < 0 || (num_peers > 0 && (!peers || !send_rows || !send_counts || !recv_rows || !recv_counts)))
            throw ArgError("halo_exchange: bad arguments");
        const NcclApi& nccl = NcclApi::get();
        size_t row_bytes = 0;
        int dtype = NcclApi::kFloat64, width = 0;
        with_halo_array(name, [&](auto* p, size_t, int w) {
            using U = std::remove_pointer_t<decltype(p)>;
            row_bytes = static_cast<size_t>(w) * sizeof(U);
            width = w;
            dtype = sizeof(U) == 4 ? NcclApi::kFloat32 : NcclApi::kFloat64;
        });
        while (static_cast<int>(xbuf_send.size()) < num_peers) {
            xbuf_send.push_back(std::make_unique<DevBuf<unsigned char>>());
            xbuf_recv.push_back(std::make_unique<DevBuf<unsigned char>>());
        }
        for (int q = 0; q < num_peers; ++q) {
            if (peers[q] < 0 || peers[q] >= comm_size || peers[q] == comm_rank || send_counts[q] < 0 || recv_counts[q] < 0)
                throw ArgError("halo_exchange: bad peer or count");
            xbuf_send[q]->resize(static_cast<size_t>(send_counts[q]) * row_bytes, stream);
            xbuf_recv[q]->resize(static_cast<size_t>(recv_counts[q]) * row_bytes, stream);
            halo_pack(name, send_rows[q], send_counts[q], xbuf_send[q]->p);
        }
        nccl.check(nccl.GroupStart(), "ncclGroupStart");
        for (int q = 0; q < num_peers; ++q) {
            if (send_counts[q] > 0)
                nccl.check(nccl.Send(xbuf_send[q]->p, static_cast<size_t>(send_counts[q]) * width, dtype, peers[q], comm, stream), "ncclSend");
            if (recv_counts[q] > 0)
                nccl.check(nccl.Recv(xbuf_recv[q]->p, static_cast<size_t>(recv_counts[q]) * width, dtype, peers[q], comm, stream), "ncclRecv");
        }
        nccl.check(nccl.GroupEnd(), "ncclGroupEnd");
        launches += 1;
        for (int q = 0; q < num_peers; ++q) halo_unpack(name, recv_rows[q], recv_counts[q], xbuf_recv[q]->p, add);
    }
    // Sum of `n` doubles (device pointer, in place) over all ranks of the communicator, on the evaluator's stream.
    void allreduce_sum(double* values, int n) override {
        SMX_CUDA(cudaSetDevice(device));
        if (!comm) throw ArgError("allreduce_sum: call smx_comm_init first");
        if (n < 0 || (n > 0 && !values)) throw ArgError("allreduce_sum: bad arguments");
        const NcclApi& nccl = NcclApi::get();
        nccl.check(nccl.AllReduce(values, values, static_cast<size_t>(n), NcclApi::kFloat64, NcclApi::kSum, comm, stream), "ncclAllReduce");
        launches += 1;
    }

    void active_counts(int* nodes, long* edges, int* built_nodes) const override {
        if (nodes) *nodes = N;
        if (edges) *edges = E;
        if (built_nodes) *built_nodes = N_built;
    }

    void reduce_forces(int rows, double* f, double* virial, double* energy, int mem_space) override {
        require_edges();
        SMX_CUDA(cudaSetDevice(device));
        if (rows < N) throw ArgError("reduce_forces: num_rows must be at least num_nodes");
        const cudaMemcpyKind kind = mem_space == SMX_DEVICE ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost;
        if (f) {
            atom_forces(rows);
            if (rows > 0) SMX_CUDA(cudaMemcpyAsync(f, atom_f.p, 3 * static_cast<size_t>(rows) * sizeof(double), kind, stream));
        }
        if (virial || energy) {
            const int blocks = std::max(1, std::min(num_sms * 4, static_cast<int>((std::max<long>(E, N) + 255) / 256)));
            partials.resize(static_cast<size_t>(blocks) * 7, stream);
            out7.resize(7, stream);
            energy_virial_partial_kernel<<<blocks, 256, 0, stream>>>(N, E, node_energies.p, xyz, node_forces.p, partials.p);
            check_launch("energy_virial_partial_kernel");
            energy_virial_final_kernel<<<1, 7 * 32, 0, stream>>>(blocks, partials.p, out7.p);
            check_launch("energy_virial_final_kernel");
            if (energy) SMX_CUDA(cudaMemcpyAsync(energy, out7.p, sizeof(double), kind, stream));
            if (virial) SMX_CUDA(cudaMemcpyAsync(virial, out7.p + 1, 6 * sizeof(double), kind, stream));
        }
        if (mem_space != SMX_DEVICE) check_kernel_status();   // device destinations: asynchronous on the stream
    }

    // ------------------------------------------------------------------ neighbour list
    long build_neighbors(int natoms, const double* pos, const int* types, const double* cell, const int* pbc, double r_cut,
                         int mem_space) override {
        SMX_CUDA(cudaSetDevice(device));
        if (natoms < 0 || (natoms > 0 && (!pos || !types)) || !cell || !pbc) throw ArgError("build_neighbors: bad arguments");
        const int* d_types = stage_input(types, natoms, in_node_types, mem_space);
        long n_edges = 0;
        nb.build(natoms, pos, d_types, cell, pbc, r_cut, mem_space == SMX_DEVICE, stream, launches, in_num_neigh, in_neigh_indices,
                 in_neigh_types, in_shifts, in_xyz, in_r, n_edges);
        node_types = d_types;
        num_neigh = in_num_neigh.p; neigh_indices = in_neigh_indices.p; neigh_types = in_neigh_types.p;
        xyz = in_xyz.p; r = in_r.p;
        N_built = natoms;
        adopt_edges(natoms, n_edges);
        SMX_CUDA(cudaStreamSynchronize(stream));
        return n_edges;
    }

    void get_edges(int* o_nn, int* o_ni, int* o_et, int* o_sh, double* o_xyz, double* o_r, int mem_space) override {
        require_edges();
        SMX_CUDA(cudaSetDevice(device));
        const cudaMemcpyKind kind = mem_space == SMX_DEVICE ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost;
        if (o_nn && N) SMX_CUDA(cudaMemcpyAsync(o_nn, num_neigh, N * sizeof(int), kind, stream));
        if (o_ni && E) SMX_CUDA(cudaMemcpyAsync(o_ni, neigh_indices, E * sizeof(int), kind, stream));
        if (o_et && E) SMX_CUDA(cudaMemcpyAsync(o_et, neigh_types, E * sizeof(int), kind, stream));
        if (o_sh && E) {
            if (in_shifts.n != 3 * static_cast<size_t>(E)) throw ArgError("get_edges: shifts exist only for edge sets built by smx_build_neighbors");
            SMX_CUDA(cudaMemcpyAsync(o_sh, in_shifts.p, 3 * E * sizeof(int), kind, stream));
        }
        if (o_xyz && E) SMX_CUDA(cudaMemcpyAsync(o_xyz, xyz, 3 * E * sizeof(double), kind, stream));
        if (o_r && E) SMX_CUDA(cudaMemcpyAsync(o_r, r, E * sizeof(double), kind, stream));
        SMX_CUDA(cudaStreamSynchronize(stream));
    }
};

// Peak fused-multiply-add rate of the SIMT pipes, measured with independent register chains.
// The edge kernels are FMA-bound, so this is the roof they are compared with.
template <typename T>
__global__ void fma_peak_kernel(T* out, int iters) {
    T a0 = T(threadIdx.x) * T(1e-3), a1 = a0 + T(1), a2 = a0 + T(2), a3 = a0 + T(3), a4 = a0 + T(4), a5 = a0 + T(5), a6 = a0 + T(6),
      a7 = a0 + T(7);
    const T b = T(0.999999), c = T(1e-7);
    for (int i = 0; i < iters; ++i) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            a0 = a0 * b + c; a1 = a1 * b + c; a2 = a2 * b + c; a3 = a3 * b + c;
            a4 = a4 * b + c; a5 = a5 * b + c; a6 = a6 * b + c; a7 = a7 * b + c;
        }
    }
    out[blockIdx.x * blockDim.x + threadIdx.x] = a0 + a1 + a2 + a3 + a4 + a5 + a6 + a7;
}

template <typename T>
double measure_fma_peak(int device) {
    SMX_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop{};
    SMX_CUDA(cudaGetDeviceProperties(&prop, device));
    const int blocks = prop.multiProcessorCount * 8, threads = 256, iters = 4096;
    T* out = nullptr;
    SMX_CUDA(cudaMalloc(&out, sizeof(T) * blocks * threads));
    cudaEvent_t e0, e1;
    SMX_CUDA(cudaEventCreate(&e0));
    SMX_CUDA(cudaEventCreate(&e1));
    double best = 0.0;
    for (int rep = 0; rep < 5; ++rep) {
        SMX_CUDA(cudaEventRecord(e0));
        fma_peak_kernel<T><<<blocks, threads>>>(out, iters);
        SMX_CUDA(cudaEventRecord(e1));
        SMX_CUDA(cudaEventSynchronize(e1));
        float ms = 0.f;
        SMX_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        const double flops = 2.0 * 64.0 * iters * double(blocks) * threads;
        best = std::max(best, flops / (ms * 1e-3) / 1e12);
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFree(out);
    return best;
}

}  // namespace smx

