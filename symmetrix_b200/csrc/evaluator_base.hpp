// Precision-independent interface of the evaluator, used by the extern "C" layer (capi.cu); the two
// instantiations of Evaluator<T> live in their own translation units so that they compile in parallel.
#pragma once

#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "model.hpp"

namespace smx {

class EvaluatorBase {
public:
    virtual ~EvaluatorBase() = default;
    HostModel model;
    int precision = 64, device = 0;
    std::string last_error;
    long launches = 0;
    double last_ms = 0.0;
    bool profiling = false;
    std::vector<std::pair<std::string, double>> stage_ms;   // per-stage device time of the last compute (profiling on)
    virtual void timer_start() = 0;
    virtual double timer_stop() = 0;
    virtual void sync() = 0;
    virtual void measure_row_stream(int layer, double* ms, double* bytes) = 0;
    virtual long validate_inputs(int feature_rows, long* counts) = 0;
    virtual void set_stream(void* s, bool external) = 0;
    virtual long restrict_nodes(int num_nodes, bool keep_outputs) = 0;
    virtual void resize_rows(const std::string& name, int rows) = 0;
    virtual void* device_ptr(const std::string& name, long* count, int* elem_bytes) = 0;

    virtual void begin(int N, const int* node_types, const int* num_neigh, const int* neigh_indices,
                       const int* neigh_types, const double* xyz, const double* r, long E, int mem_space) = 0;
    virtual void stage(const std::string& name, bool zero_dxyz, bool zero_H1_adj) = 0;
    virtual void compute_all() = 0;
    virtual long get_array(const std::string& name, double* dst, long cap, int mem_space) = 0;
    virtual void set_array(const std::string& name, const double* src, long n, int mem_space) = 0;
    virtual void reduce_forces(int rows, double* f, double* virial, double* energy, int mem_space) = 0;
    virtual void atom_forces(int rows) = 0;
    virtual void halo_pack(const std::string& name, const int* rows, int n, void* dst) = 0;
    virtual void halo_unpack(const std::string& name, const int* rows, int n, const void* src, bool add) = 0;
    virtual void expire_waits(int polls) = 0;
    virtual void halo_cache_lists(int enable) = 0;
    virtual void comm_init(const void* id, int id_bytes, int nranks, int rank) = 0;
    virtual void comm_destroy() = 0;
    virtual void halo_exchange(const std::string& name, bool add, int num_peers, const int* peers, const int* const* send_rows,
                               const int* send_counts, const int* const* recv_rows, const int* recv_counts) = 0;
    virtual void allreduce_sum(double* values, int n) = 0;
    virtual void active_counts(int* nodes, long* edges, int* built_nodes) const = 0;
    virtual long build_neighbors(int natoms, const double* pos, const int* types, const double* cell, const int* pbc,
                                 double r_cut, int mem_space) = 0;
    virtual void get_edges(int* num_neigh, int* neigh_indices, int* neigh_types, int* shifts, double* xyz, double* r, int mem_space) = 0;
};

std::unique_ptr<EvaluatorBase> make_evaluator_f32(HostModel&& m, int device);
std::unique_ptr<EvaluatorBase> make_evaluator_f64(HostModel&& m, int device);
double measure_fma_peak_f32(int device);
double measure_fma_peak_f64(int device);

}  // namespace smx
