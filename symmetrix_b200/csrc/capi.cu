// The extern "C" entry points declared in include/symmetrix_b200.h: argument checks, exception -> status code,
// and dispatch to the evaluator of the handle's precision.
#include <cuda_runtime.h>

#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>

#include "../../include/symmetrix_b200.h"
#include "common.cuh"
#include "evaluator_base.hpp"
#include "model_cache.hpp"
#include "nccl_transport.hpp"

// =================================================================================================
// extern "C" entry points
// =================================================================================================
struct smx_evaluator {
    std::unique_ptr<smx::EvaluatorBase> impl;
};

namespace {
thread_local std::string g_create_error;

template <typename Fn>
int guarded(smx_handle h, Fn&& fn) {
    if (!h || !h->impl) return SMX_ERR_INVALID_ARGUMENT;
    try {
        fn(*h->impl);
        return SMX_OK;
    } catch (const smx::ArgError& e) {
        h->impl->last_error = e.what();
        return SMX_ERR_INVALID_ARGUMENT;
    } catch (const smx::UnsupportedError& e) {
        h->impl->last_error = e.what();
        return SMX_ERR_UNSUPPORTED;
    } catch (const smx::CudaError& e) {
        h->impl->last_error = e.what();
        return SMX_ERR_CUDA;
    } catch (const std::exception& e) {
        h->impl->last_error = e.what();
        return SMX_ERR_INVALID_ARGUMENT;
    }
}
}  // namespace

extern "C" {

int smx_create(const char* json_path, int precision, int device, smx_handle* out) {
    if (!out) return SMX_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    try {
        if (!json_path) throw smx::ArgError("smx_create: null path");
        if (precision != SMX_FP32 && precision != SMX_FP64) throw smx::ArgError("smx_create: precision must be 32 or 64");
        // the model is read and validated first, so a bad file is reported as such on any machine
        smx::HostModel m = smx::load_model_cached(json_path);
        int count = 0;
        if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
            cudaGetLastError();
            g_create_error = "no CUDA device available: this library has no CPU path";
            return SMX_ERR_NO_DEVICE;
        }
        if (device < 0 || device >= count) throw smx::ArgError("smx_create: device ordinal out of range");
        auto h = std::make_unique<smx_evaluator>();
        if (precision == SMX_FP32) h->impl = smx::make_evaluator_f32(std::move(m), device);
        else h->impl = smx::make_evaluator_f64(std::move(m), device);
        *out = h.release();
        return SMX_OK;
    } catch (const smx::ArgError& e) { g_create_error = e.what(); return SMX_ERR_INVALID_ARGUMENT;
    } catch (const smx::UnsupportedError& e) { g_create_error = e.what(); return SMX_ERR_UNSUPPORTED;
    } catch (const smx::CudaError& e) { g_create_error = e.what(); return SMX_ERR_CUDA;
    } catch (const std::exception& e) { g_create_error = e.what(); return SMX_ERR_MODEL; }  // JsonError, ModelError, I/O
}

void smx_destroy(smx_handle h) { delete h; }

const char* smx_last_error(smx_handle h) {
    if (!h || !h->impl) return g_create_error.c_str();
    return h->impl->last_error.c_str();
}

int smx_info(smx_handle h, smx_model_info* info) {
    if (!info) return SMX_ERR_INVALID_ARGUMENT;
    return guarded(h, [&](smx::EvaluatorBase& e) {
        const smx::HostModel& m = e.model;
        info->num_elements = m.num_elements; info->num_channels = m.K; info->r_cut = m.r_cut;
        info->l_max = m.l_max; info->num_lm = m.num_lm; info->L_max = m.L_max; info->num_LM = m.num_LM;
        info->num_paths = m.tp.P; info->num_lelm1lm2 = m.tp.T; info->num_lme = m.tp.Q;
        info->num_interactions = m.num_interactions;
        info->has_zbl = m.has_zbl ? 1 : 0; info->precision = e.precision; info->device = e.device;
    });
}

int smx_atomic_numbers(smx_handle h, int* out, int cap) {
    if (!h || !h->impl) return -1;
    const auto& v = h->impl->model.atomic_numbers;
    for (int i = 0; i < static_cast<int>(v.size()) && i < cap && out; ++i) out[i] = v[i];
    return static_cast<int>(v.size());
}
int smx_atomic_energies(smx_handle h, double* out, int cap) {
    if (!h || !h->impl) return -1;
    const auto& v = h->impl->model.atomic_energies;
    for (int i = 0; i < static_cast<int>(v.size()) && i < cap && out; ++i) out[i] = v[i];
    return static_cast<int>(v.size());
}

int smx_begin(smx_handle h, int num_nodes, const int* node_types, const int* num_neigh, const int* neigh_indices,
              const int* neigh_types, const double* xyz, const double* r, long num_edges, int mem_space) {
    return guarded(h, [&](smx::EvaluatorBase& e) {
        e.begin(num_nodes, node_types, num_neigh, neigh_indices, neigh_types, xyz, r, num_edges, mem_space);
    });
}

int smx_compute(smx_handle h, int num_nodes, const int* node_types, const int* num_neigh, const int* neigh_indices,
                const int* neigh_types, const double* xyz, const double* r, long num_edges, int mem_space) {
    return guarded(h, [&](smx::EvaluatorBase& e) {
        e.begin(num_nodes, node_types, num_neigh, neigh_indices, neigh_types, xyz, r, num_edges, mem_space);
        e.compute_all();
    });
}

int smx_compute_current(smx_handle h) {
    return guarded(h, [&](smx::EvaluatorBase& e) { e.compute_all(); });
}

int smx_stage(smx_handle h, const char* name, int zero_dxyz, int zero_H1_adj) {
    return guarded(h, [&](smx::EvaluatorBase& e) {
        if (!name) throw smx::ArgError("smx_stage: null name");
        e.stage(name, zero_dxyz != 0, zero_H1_adj != 0);
    });
}

int smx_get_array(smx_handle h, const char* name, double* dst, long cap, long* n, int mem_space) {
    return guarded(h, [&](smx::EvaluatorBase& e) {
        if (!name) throw smx::ArgError("smx_get_array: null name");
        const long count = e.get_array(name, dst, cap, mem_space);
        if (n) *n = count;
    });
}

int smx_set_array(smx_handle h, const char* name, const double* src, long n, int mem_space) {
    return guarded(h, [&](smx::EvaluatorBase& e) {
        if (!name) throw smx::ArgError("smx_set_array: null name");
        e.set_array(name, src, n, mem_space);
    });
}

int smx_reduce_forces(smx_handle h, int num_rows, double* atom_forces, double* virial, double* energy, int mem_space) {
    return guarded(h, [&](smx::EvaluatorBase& e) { e.reduce_forces(num_rows, atom_forces, virial, energy, mem_space); });
}

int smx_atom_forces(smx_handle h, int num_rows) {
    return guarded(h, [&](smx::EvaluatorBase& e) { e.atom_forces(num_rows); });
}

int smx_halo_pack(smx_handle h, const char* name, const int* rows, int n, void* dst) {
    return guarded(h, [&](smx::EvaluatorBase& e) {
        if (!name) throw smx::ArgError("smx_halo_pack: null name");
        e.halo_pack(name, rows, n, dst);
    });
}
int smx_halo_unpack(smx_handle h, const char* name, const int* rows, int n, const void* src) {
    return guarded(h, [&](smx::EvaluatorBase& e) {
        if (!name) throw smx::ArgError("smx_halo_unpack: null name");
        e.halo_unpack(name, rows, n, src, false);
    });
}
int smx_halo_unpack_add(smx_handle h, const char* name, const int* rows, int n, const void* src) {
    return guarded(h, [&](smx::EvaluatorBase& e) {
        if (!name) throw smx::ArgError("smx_halo_unpack_add: null name");
        e.halo_unpack(name, rows, n, src, true);
    });
}
int smx_model_digest(const char* json_path, int use_cache, unsigned long long* digest, int* from_cache) {
    try {
        if (!json_path || !digest) throw smx::ArgError("smx_model_digest: null argument");
        bool hit = false;
        smx::HostModel m = use_cache ? smx::load_model_cached(json_path, &hit) : smx::load_model_file(json_path);
        *digest = smx::model_digest(m);
        if (from_cache) *from_cache = hit ? 1 : 0;
        return SMX_OK;
    } catch (const smx::ArgError& e) { g_create_error = e.what(); return SMX_ERR_INVALID_ARGUMENT;
    } catch (const smx::UnsupportedError& e) { g_create_error = e.what(); return SMX_ERR_UNSUPPORTED;
    } catch (const std::exception& e) { g_create_error = e.what(); return SMX_ERR_MODEL; }
}

int smx_comm_unique_id(void* id, int id_bytes) {
    try {
        if (!id || id_bytes != static_cast<int>(sizeof(smx::NcclApi::UniqueId))) throw smx::ArgError("smx_comm_unique_id: the id buffer must hold 128 bytes");
        const smx::NcclApi& nccl = smx::NcclApi::get();
        smx::NcclApi::UniqueId uid;
        nccl.check(nccl.GetUniqueId(&uid), "ncclGetUniqueId");
        std::memcpy(id, &uid, sizeof(uid));
        return SMX_OK;
    } catch (const smx::ArgError& e) { g_create_error = e.what(); return SMX_ERR_INVALID_ARGUMENT;
    } catch (const std::exception& e) { g_create_error = e.what(); return SMX_ERR_CUDA; }
}
int smx_comm_init(smx_handle h, const void* id, int id_bytes, int num_ranks, int rank) {
    return guarded(h, [&](smx::EvaluatorBase& e) { e.comm_init(id, id_bytes, num_ranks, rank); });
}
int smx_comm_destroy(smx_handle h) {
    return guarded(h, [&](smx::EvaluatorBase& e) { e.comm_destroy(); });
}
int smx_halo_exchange(smx_handle h, const char* name, int add, int num_peers, const int* peers, const int* const* send_rows,
                      const int* send_counts, const int* const* recv_rows, const int* recv_counts) {
    return guarded(h, [&](smx::EvaluatorBase& e) {
        if (!name) throw smx::ArgError("smx_halo_exchange: null name");
        e.halo_exchange(name, add != 0, num_peers, peers, send_rows, send_counts, recv_rows, recv_counts);
    });
}
int smx_allreduce_sum(smx_handle h, double* values, int n) {
    return guarded(h, [&](smx::EvaluatorBase& e) { e.allreduce_sum(values, n); });
}
int smx_active_counts(smx_handle h, int* num_nodes, long* num_edges, int* built_nodes) {
    return guarded(h, [&](smx::EvaluatorBase& e) { e.active_counts(num_nodes, num_edges, built_nodes); });
}
int smx_halo_cache_lists(smx_handle h, int enable) {
    return guarded(h, [&](smx::EvaluatorBase& e) { e.halo_cache_lists(enable); });
}
int smx_debug_expire_waits(smx_handle h, int polls) {
    return guarded(h, [&](smx::EvaluatorBase& e) { e.expire_waits(polls); });
}

int smx_last_device_ms(smx_handle h, double* ms) {
    return guarded(h, [&](smx::EvaluatorBase& e) { if (ms) *ms = e.last_ms; });
}

long smx_launch_count(smx_handle h) { return (h && h->impl) ? h->impl->launches : -1; }

int smx_sync(smx_handle h) {
    return guarded(h, [&](smx::EvaluatorBase& e) { e.sync(); });
}
int smx_set_stream(smx_handle h, void* stream, int external) {
    return guarded(h, [&](smx::EvaluatorBase& e) { e.set_stream(stream, external != 0); });
}
int smx_restrict_nodes(smx_handle h, int num_nodes, long* num_edges) {
    return guarded(h, [&](smx::EvaluatorBase& e) { const long n = e.restrict_nodes(num_nodes, false); if (num_edges) *num_edges = n; });
}

int smx_set_active_nodes(smx_handle h, int num_nodes, long* num_edges) {
    return guarded(h, [&](smx::EvaluatorBase& e) { const long n = e.restrict_nodes(num_nodes, true); if (num_edges) *num_edges = n; });
}
int smx_resize_rows(smx_handle h, const char* name, int rows) {
    return guarded(h, [&](smx::EvaluatorBase& e) {
        if (!name) throw smx::ArgError("smx_resize_rows: null name");
        e.resize_rows(name, rows);
    });
}
int smx_device_ptr(smx_handle h, const char* name, void** ptr, long* count, int* elem_bytes) {
    return guarded(h, [&](smx::EvaluatorBase& e) {
        if (!name || !ptr) throw smx::ArgError("smx_device_ptr: null argument");
        *ptr = e.device_ptr(name, count, elem_bytes);
    });
}
int smx_timer_start(smx_handle h) {
    return guarded(h, [&](smx::EvaluatorBase& e) { e.timer_start(); });
}
int smx_timer_stop(smx_handle h, double* ms) {
    return guarded(h, [&](smx::EvaluatorBase& e) { const double t = e.timer_stop(); if (ms) *ms = t; });
}
int smx_set_profiling(smx_handle h, int enabled) {
    return guarded(h, [&](smx::EvaluatorBase& e) { e.profiling = enabled != 0; });
}
int smx_stage_time(smx_handle h, int index, char* name, int name_cap, double* ms) {
    return guarded(h, [&](smx::EvaluatorBase& e) {
        if (index < 0 || index >= static_cast<int>(e.stage_ms.size())) throw smx::ArgError("smx_stage_time: index out of range");
        if (name && name_cap > 0) {
            std::strncpy(name, e.stage_ms[index].first.c_str(), name_cap - 1);
            name[name_cap - 1] = 0;
        }
        if (ms) *ms = e.stage_ms[index].second;
    });
}

int smx_measure_fma_peak(int precision, int device, double* tflops) {
    try {
        if (!tflops) throw smx::ArgError("null output");
        *tflops = precision == SMX_FP32 ? smx::measure_fma_peak_f32(device) : smx::measure_fma_peak_f64(device);
        return SMX_OK;
    } catch (const std::exception& e) {
        g_create_error = e.what();
        return SMX_ERR_CUDA;
    }
}

int smx_measure_row_stream(smx_handle h, int layer, double* ms, double* bytes) {
    return guarded(h, [&](smx::EvaluatorBase& e) { e.measure_row_stream(layer, ms, bytes); });
}

int smx_validate_inputs(smx_handle h, int feature_rows, long* counts, long* total) {
    return guarded(h, [&](smx::EvaluatorBase& e) {
        const long n = e.validate_inputs(feature_rows, counts);
        if (total) *total = n;
        if (n != 0) throw smx::ArgError("the edge arrays hold " + std::to_string(n) + " out-of-range or inconsistent entries");
    });
}

int smx_build_neighbors(smx_handle h, int num_atoms, const double* positions, const int* types, const double* cell,
                        const int* pbc, double r_cut, long* num_edges, int mem_space) {
    return guarded(h, [&](smx::EvaluatorBase& e) {
        const long n = e.build_neighbors(num_atoms, positions, types, cell, pbc, r_cut, mem_space);
        if (num_edges) *num_edges = n;
    });
}

int smx_get_edges(smx_handle h, int* num_neigh, int* neigh_indices, int* neigh_types, int* shifts, double* xyz, double* r,
                  int mem_space) {
    return guarded(h, [&](smx::EvaluatorBase& e) { e.get_edges(num_neigh, neigh_indices, neigh_types, shifts, xyz, r, mem_space); });
}

}  // extern "C"
