/* symmetrix_b200 -- C ABI of the B200-native MACE energy+force evaluator.
 *
 * This is the drop-in boundary for the evaluation path of wcwitt/symmetrix: every entry
 * point below replaces one piece of the reference's `class MACE` (CPU) /
 * `class MACEKokkos<Precision>` (device) interface, which is what the reference's pybind11
 * module and its LAMMPS pair style bind. Plain pointers and sizes only; no C++ or torch
 * types cross this boundary. All functions return 0 on success and a non-zero status
 * otherwise; the message is then available from smx_last_error(). Nothing throws.
 *
 * Conventions shared by all calls
 *  - `mem_space` says where the caller's arrays live: SMX_HOST or SMX_DEVICE (pointers valid
 *    on the evaluator's device). Host arrays are copied in/out by the library.
 *  - Edges are grouped by receiver node (CSR): node i owns `num_neigh[i]` consecutive edges.
 *    `neigh_indices[e]` is the row of the sender's features, `xyz[3e..3e+2] = x_j - x_i`,
 *    `r[e] = |xyz_e|`. This is exactly the argument list of the reference
 *    (libsymmetrix/source/mace.hpp:28-36).
 *  - Work is issued on the evaluator's own CUDA stream; calls return after the stream has
 *    been synchronised when any output goes to host memory.
 *  - One evaluator per GPU and per host thread; an evaluator is not thread-safe (neither is
 *    the reference: all scratch is per-object state, mace.hpp:40-164).
 */
#ifndef SYMMETRIX_B200_H
#define SYMMETRIX_B200_H

#ifdef __cplusplus
extern "C" {
#endif

typedef struct smx_evaluator* smx_handle;

enum { SMX_HOST = 0, SMX_DEVICE = 1 };
enum { SMX_FP32 = 32, SMX_FP64 = 64 };

enum {
    SMX_OK = 0,
    SMX_ERR_INVALID_ARGUMENT = 1, /* bad size, unknown name, null pointer                     */
    SMX_ERR_MODEL = 2,            /* model file missing, not JSON, or outside the supported set */
    SMX_ERR_CUDA = 3,             /* a CUDA runtime call or kernel launch failed               */
    SMX_ERR_UNSUPPORTED = 4,      /* feature of the reference that this build does not cover   */
    SMX_ERR_NO_DEVICE = 5         /* no usable CUDA device: there is no CPU fallback           */
};

typedef struct smx_model_info {
    int num_elements;   /* MACE::num_elements  (mace.hpp:19) */
    int num_channels;   /* MACE::num_channels  (mace.hpp:20) */
    double r_cut;       /* MACE::r_cut         (mace.hpp:21) */
    int l_max, num_lm;  /* MACE::l_max, num_lm (mace.hpp:22) */
    int L_max, num_LM;  /* MACE::L_max, num_LM (mace.hpp:23) */
    int num_paths;      /* number of tensor-product paths, Phi1_l.size() (mace.hpp:115)      */
    int num_lelm1lm2;   /* MACE::num_lelm1lm2  (mace.hpp:112) */
    int num_lme;        /* MACE::num_lme       (mace.hpp:112) */
    int has_zbl;        /* MACE::has_zbl       (mace.hpp:39)  */
    int precision;      /* SMX_FP32 or SMX_FP64: arithmetic type of features and weights     */
    int device;         /* CUDA device ordinal the evaluator lives on                        */
    int num_interactions; /* 2 (every model the reference can export) or 3 (file key "num_interactions") */
} smx_model_info;

/* Replaces the constructor MACE::MACE(std::string filename) -> load_from_json
 * (libsymmetrix/source/mace.cpp:12-15,905-1030; device twin mace_kokkos.cpp:1544-1887).
 * `precision` selects what MACEKokkos<float> / MACEKokkos<double> select in the reference
 * (symmetrix/source/symmetrix/symmetrix_calc.py:49). Fails with SMX_ERR_NO_DEVICE when no GPU
 * is present. */
int smx_create(const char* json_path, int precision, int device, smx_handle* out);

/* Replaces the destructor of MACE / MACEKokkos. */
void smx_destroy(smx_handle h);

/* Message of the last failing call on `h` (or of the last failing smx_create when h is NULL).
 * Stands in for the C++ exceptions the reference reports errors with
 * (e.g. cubic_spline.cpp:19-20; nlohmann parse_error surfacing in symmetrix_calc.py:54-68). */
const char* smx_last_error(smx_handle h);

/* Replaces reads of the public data members num_elements, num_channels, r_cut, l_max, num_lm,
 * L_max, num_LM, has_zbl (mace.hpp:18-39). */
int smx_info(smx_handle h, smx_model_info* info);

/* Replaces reads of MACE::atomic_numbers / MACE::atomic_energies (mace.hpp:24-25), which the
 * pair style and the ASE calculator use to map species to model types
 * (pair_symmetrix/pair_symmetrix_mace.cpp:122-138; symmetrix_calc.py:75-81). `cap` is the
 * capacity of `out`; the return value is the number of elements of the model. */
int smx_atomic_numbers(smx_handle h, int* out, int cap);
int smx_atomic_energies(smx_handle h, double* out, int cap);

/* Replaces MACE::compute_node_energies_forces (libsymmetrix/source/mace.cpp:17-64; device twin
 * mace_kokkos.cpp:49-98): zero the outputs, run all forward stages, the readouts and all reverse
 * stages. Results stay on the device and are read with smx_get_array("node_energies" /
 * "node_forces") or reduced with smx_reduce_forces. */
int smx_compute(smx_handle h, int num_nodes, const int* node_types, const int* num_neigh,
                const int* neigh_indices, const int* neigh_types, const double* xyz,
                const double* r, long num_edges, int mem_space);

/* Replaces the individual stage methods of MACE that the message-passing pair-style mode calls
 * one by one (mace.hpp:40-164; call sequence pair_symmetrix/pair_symmetrix_mace.cpp:444-495):
 * name is one of compute_Y, compute_R0, compute_A0, compute_M0, compute_H1, compute_R1,
 * compute_Phi1, compute_A1, compute_M1, compute_H2, compute_readouts, reverse_H2, reverse_M1,
 * reverse_A1, reverse_Phi1, reverse_H1, reverse_M0, reverse_A0, compute_ZBL (ZBL::compute_ZBL,
 * zbl.hpp:29-37, a no-op for models without pair repulsion) and compute_A0_scaled, compute_A1_scaled,
 * reverse_A0_scaled, reverse_A1_scaled (no-ops for models without density normalisation, as in the
 * reference). `zero_dxyz` / `zero_H1_adj` carry the flags of reverse_Phi1 / reverse_H2 /
 * reverse_A1_scaled (mace.hpp:118,145,159).
 * Models whose file says "num_interactions": 3 (an extension; the reference's exporter stops at two blocks,
 * extract_mace_data.py:70-71) add compute_Rm (no-op), compute_Phim, compute_Am, compute_Mm, compute_Hm between
 * compute_H1 and compute_R1, and reverse_Hm, reverse_Mm, reverse_Am, reverse_Phim between reverse_Phi1 and
 * reverse_H1: the stages of a second interaction block whose contraction keeps every (L, M); the arrays Phim, Am,
 * Mm, Hm and their adjoints are read and written like the others, and Hm / Hm_adj take ghost rows like H1 / H1_adj.
 * Radial functions and harmonics are recomputed inside the edge kernels, so compute_Y /
 * compute_R0 / compute_R1 only record the edge arrays they are given. A sequence of stage calls
 * must start with smx_begin, which replaces the zero-fill of node_energies / node_forces that
 * callers do by hand (pair_symmetrix_mace.cpp:437-440). */
int smx_begin(smx_handle h, int num_nodes, const int* node_types, const int* num_neigh,
              const int* neigh_indices, const int* neigh_types, const double* xyz,
              const double* r, long num_edges, int mem_space);
int smx_stage(smx_handle h, const char* name, int zero_dxyz, int zero_H1_adj);

/* Replaces reads of the public result / intermediate vectors of MACE (node_energies,
 * node_forces, A0, A0_adj, M0, M0_adj, H1, H1_adj, Phi1, Phi1_adj, A1, A1_adj, M1, M1_adj, H2,
 * H2_adj: symmetrix/source/cpp/mace.cpp:14-33) -- copies `name` to `dst` as doubles.
 * `*n` receives the number of elements; at most `cap` are written. */
int smx_get_array(smx_handle h, const char* name, double* dst, long cap, long* n, int mem_space);

/* Replaces writes to those members; the message-passing mode swaps H1 / H1_adj in and out with
 * rows for ghost atoms appended (pair_symmetrix_mace.cpp:463-471,488-490). `n` may exceed the
 * current length (the array grows, as std::vector assignment does). */
int smx_set_array(smx_handle h, const char* name, const double* src, long n, int mem_space);

/* Replaces the force / energy / virial reduction every caller performs on the per-edge partial
 * forces: f[i] -= nf_ij, f[j] += nf_ij, virial += sym(xyz_ij (x) nf_ij), energy = sum of node
 * energies (pair_symmetrix/pair_symmetrix_mace.cpp:324-368; symmetrix_calc.py:85-102).
 * `atom_forces` has 3*num_rows doubles with num_rows >= 1 + max(neigh_indices); `virial` has 6
 * (xx, yy, zz, xy, xz, yz). Any output pointer may be NULL. Deterministic (no atomics). With
 * host destinations the call returns when the results are there; with device destinations it is
 * asynchronous on the evaluator's stream. */
int smx_reduce_forces(smx_handle h, int num_rows, double* atom_forces, double* virial,
                      double* energy, int mem_space);

/* Milliseconds spent on the device by the last smx_compute (CUDA events on the evaluator's
 * stream). The reference has no counterpart; the Kokkos build relies on external tools. */
int smx_last_device_ms(smx_handle h, double* ms);

/* Number of kernels the evaluator launched since creation (for benchmark bookkeeping). */
long smx_launch_count(smx_handle h);

/* Measurement helpers; none has a counterpart in the reference (its Kokkos kernels only carry
 * labels for external tools, e.g. mace_kokkos.cpp:866). smx_timer_start/stop bracket any sequence
 * of calls with CUDA events on the evaluator's stream and return the elapsed device time.
 * With profiling on, smx_compute additionally records one event per stage, and smx_stage_time
 * returns the name and device time of stage `index` (0..14, or 0..22 for a three-block model, in execution order) of the last
 * smx_compute. smx_measure_fma_peak runs a register-only FMA loop and returns the SIMT
 * fused-multiply-add rate in TFLOP/s, the roof of the FMA-bound edge kernels.
 * smx_measure_row_stream runs, over the evaluator's current edge set, a kernel that only reads the
 * spline row of every edge from the table of interaction layer `layer` (0 or 1) the way the edge
 * kernels do; it returns its device time and the bytes read, the floor that streaming the
 * coefficients from L2 sets for one pass of an edge kernel. */
int smx_timer_start(smx_handle h);
int smx_timer_stop(smx_handle h, double* ms);
int smx_set_profiling(smx_handle h, int enabled);
int smx_stage_time(smx_handle h, int index, char* name, int name_cap, double* ms);
int smx_measure_fma_peak(int precision, int device, double* tflops);
int smx_measure_row_stream(smx_handle h, int layer, double* ms, double* bytes);

/* Neighbour list on the device -- replaces, for callers without their own, the external
 * builders the reference's callers rely on: ase/matscipy `neighbor_list('ijdD', atoms, r_cut)`
 * (symmetrix_calc.py:12-16,77) and the LAMMPS full list filtered by r^2 < r_cut^2
 * (pair_symmetrix_mace.cpp:249-315). Edge rule, float64 arithmetic and ordering are stated in
 * symmetrix_b200/structures.py::neighbor_list, which is the host statement of the same rule.
 * Builds the CSR arrays of the evaluator for `num_atoms` atoms in a periodic cell (row vectors
 * `cell[9]`, `pbc[3]`), keeps them on the device as the current edge set (as smx_begin does)
 * and returns the edge count. `types[i]` is the model type of atom i. */
int smx_build_neighbors(smx_handle h, int num_atoms, const double* positions, const int* types,
                        const double* cell, const int* pbc, double r_cut, long* num_edges,
                        int mem_space);
/* Copies out the edge arrays of the current edge set (any pointer may be NULL). */
int smx_get_edges(smx_handle h, int* num_neigh, int* neigh_indices, int* neigh_types,
                  int* shifts, double* xyz, double* r, int mem_space);
/* smx_compute on the current edge set (after smx_build_neighbors). */
int smx_compute_current(smx_handle h);

/* Helpers for callers that decompose a structure across GPUs and exchange halo rows on the device
 * (the role LAMMPS' Comm plays for the reference's message-passing mode, pair_symmetrix_mace.cpp:
 * 194-238,463-490 -- there the rows travel through host vectors and MPI).
 * smx_sync waits for the evaluator's stream; smx_set_stream makes the evaluator issue all further work on the
 * caller's cudaStream_t when `external` is non-zero (a NULL handle then means the legacy default stream) and
 * returns to its own stream when `external` is zero, so that pack / unpack kernels and NCCL calls of the
 * caller are ordered with the evaluator's kernels without host synchronisation. smx_restrict_nodes keeps only the first `num_nodes`
 * receivers of the current edge set (owned atoms first, ghost atoms after them) and returns the
 * remaining edge count; it starts a new evaluation (outputs zero-filled) and `num_nodes` may be anything up to
 * the receiver count the edge set was given or built with. smx_set_active_nodes changes the active
 * receivers the same way but in the middle of an evaluation: node energies, partial forces and feature
 * rows beyond the active nodes are kept. That is the reference's recompute mode
 * (pair_symmetrix_mace.cpp:551-748), where layer 0 and its reverse run on owned + ghost atoms
 * (MACE::compute_* called with `nlocal + nghost`-sized lists there) and layer 1 on owned atoms only.
 * smx_resize_rows grows "H1" or "H1_adj" to `rows` feature rows, keeping the
 * computed rows and zero-filling the appended ghost rows. smx_device_ptr returns the device address,
 * element count and element size (4 or 8 bytes) of a named array so that pack / unpack kernels and
 * NCCL can work on it in place; the pointer is valid until the next call that resizes that array. */
int smx_sync(smx_handle h);
int smx_set_stream(smx_handle h, void* stream, int external);
int smx_restrict_nodes(smx_handle h, int num_nodes, long* num_edges);
int smx_set_active_nodes(smx_handle h, int num_nodes, long* num_edges);
int smx_resize_rows(smx_handle h, const char* name, int rows);
int smx_device_ptr(smx_handle h, const char* name, void** ptr, long* count, int* elem_bytes);

/* Halo rows as device kernels on the evaluator's stream -- the pack / unpack routines of the reference's pair style:
 * pack_forward_comm / unpack_forward_comm / pack_reverse_comm / unpack_reverse_comm (pair_symmetrix_mace.cpp:194-238)
 * and their device forms (pair_symmetrix_mace_kokkos.cpp:240-290, 351-367). `name` is "H1", "H1_adj", "Hm", "Hm_adj"
 * (rows of num_LM * num_channels values in the evaluator's precision) or "atom_forces" (rows of 3 doubles, the array
 * smx_atom_forces fills). `rows` (n row indices) and the buffers are device pointers; a buffer holds n rows in the
 * array's own element type.
 *   smx_halo_pack        buf[m, :] = array[rows[m], :]
 *   smx_halo_unpack      array[rows[m], :] = buf[m, :]
 *   smx_halo_unpack_add  array[rows[m], :] += buf[m, :], each row's contributions added in list order by one thread --
 *                        the reference uses atomic adds here (pair_symmetrix_mace_kokkos.cpp:362-364); this one gives the
 *                        same bits on every run, also when a row occurs more than once in the list.
 * smx_atom_forces computes the per-atom forces of the current edge set (f[i] -= nf[ij], f[j] += nf[ij],
 * pair_symmetrix_mace.cpp:334-347) into the device array "atom_forces" with at least `num_rows` rows, without copying
 * them anywhere; smx_reduce_forces is this plus the copy to the caller. */
int smx_halo_pack(smx_handle h, const char* name, const int* rows, int n, void* buf);
int smx_halo_unpack(smx_handle h, const char* name, const int* rows, int n, const void* buf);
int smx_halo_unpack_add(smx_handle h, const char* name, const int* rows, int n, const void* buf);
/* smx_halo_unpack_add (and smx_halo_exchange with add) first groups the list positions by destination row: a sort per
 * call. LAMMPS rebuilds its send lists only when it re-neighbours (Comm::borders), and between those steps the pair
 * style's unpack_reverse_comm sees the same list every time (pair_symmetrix_mace_kokkos.cpp:351-367). With enable != 0 the
 * grouping of a list is kept and reused whenever a list with the same device address and length is passed again; the
 * caller promises not to change such a list in place. enable = 0 drops all kept groupings and stops keeping them (call it
 * when the lists are rebuilt, then enable again). Off by default. */
int smx_halo_cache_lists(smx_handle h, int enable);
int smx_atom_forces(smx_handle h, int num_rows);

/* Model loading with a binary side-car. MACE::load_from_json (mace.cpp:905-1030) parses the JSON text on every start;
 * smx_create does that once per model file and then reads `<file>.smxcache`, the parsed and re-laid-out tables, written
 * next to the file (a 314 MB file: 3.3 s of parsing against a fraction of a second). The side-car is valid only for the
 * exact source file (size, modification time) and the exact build of this library, is rewritten when either changes,
 * and is never required: without write permission, or with SMX_MODEL_CACHE=0 in the environment, the text is parsed.
 * smx_model_digest loads a model file (through the side-car when `use_cache` is non-zero) and returns a 64-bit FNV-1a
 * digest of everything the loader produced, so that a caller -- or a test -- can check that both routes give the same
 * model; `from_cache` (may be NULL) tells which route was taken. It needs no GPU. */
int smx_model_digest(const char* json_path, int use_cache, unsigned long long* digest, int* from_cache);

/* Halo exchange between the ranks of a decomposed run, inside the library: what LAMMPS' Comm does for the reference's
 * message-passing mode (comm->forward_comm(this) / comm->reverse_comm(this), pair_symmetrix_mace.cpp:470,489, with the pack /
 * unpack routines above) as grouped ncclSend / ncclRecv on the evaluator's stream. NCCL is loaded at run time
 * (dlopen "libnccl.so.2"), so a process that never calls these needs none. One rank obtains a 128-byte id with
 * smx_comm_unique_id and distributes it by any means (MPI_Bcast, a file, torch.distributed); every rank then calls
 * smx_comm_init(h, id, 128, num_ranks, rank) once (collective). smx_halo_exchange does one exchange with `num_peers`
 * neighbours: for peer q it packs the rows send_rows[q][0..send_counts[q]) of array `name`, sends them to rank peers[q],
 * receives recv_counts[q] rows from it and unpacks them into rows recv_rows[q][...] -- overwriting them (`add` == 0: forward
 * exchange of "H1" / "Hm") or adding in a fixed order (`add` != 0: reverse exchange of "H1_adj" / "Hm_adj" / "atom_forces").
 * The row lists are device pointers (the outer arrays of pointers and the counts are host arrays); nothing synchronises
 * with the host. smx_allreduce_sum sums `n` doubles (device pointer, in place) over all ranks: energy and virial. */
int smx_comm_unique_id(void* id, int id_bytes);
int smx_comm_init(smx_handle h, const void* id, int id_bytes, int num_ranks, int rank);
int smx_comm_destroy(smx_handle h);
int smx_halo_exchange(smx_handle h, const char* name, int add, int num_peers, const int* peers, const int* const* send_rows,
                      const int* send_counts, const int* const* recv_rows, const int* recv_counts);
int smx_allreduce_sum(smx_handle h, double* values, int n);

/* Receivers and edges the stages currently run on, and the receiver count the edge set was given or built with. The
 * reference's stage methods take `num_nodes` and the neighbour arrays on every call (mace.hpp:44-145); here they are
 * fixed by smx_begin / smx_restrict_nodes / smx_set_active_nodes, and a caller that mirrors the reference's argument
 * lists checks its `num_nodes` against this. Any pointer may be NULL. */
int smx_active_counts(smx_handle h, int* num_nodes, long* num_edges, int* built_nodes);

/* Test switch for the bounded device-side waits (no counterpart in the reference, which has no such waits). With
 * `polls` > 0 the first weight-tile wait of every CTA of the float32 tensor-core GEMM expects 16 bytes more than
 * its copy delivers and gives up after `polls` polls: the kernel records the failure, releases its tensor memory and
 * returns, and the next synchronising call reports SMX_ERR_CUDA. Nothing faults and the handle stays usable; 0 switches
 * it off. */
int smx_debug_expire_waits(smx_handle h, int polls);

/* Input check. The reference trusts its callers (unchecked spline bin and gather indices, cubic_spline_set.cpp:31-32,
 * 55-56; mace.cpp:470-480); on a GPU an out-of-range sender index is a memory fault, so callers that cannot vouch for
 * their arrays call this after smx_begin / smx_build_neighbors and before the first stage. It counts, per kind, the
 * entries of the current edge set that are out of range or inconsistent: counts[0] node type outside the model,
 * [1] negative neighbour count, [2] neighbour counts not adding up to the number of edges, [3] sender index outside
 * [0, feature_rows), [4] sender type outside the model, [5] r not finite, <= 0 or beyond r_cut, [6] r differing from
 * |xyz| by more than 1e-6 relative. `counts` (7 entries) and `total` may be NULL. Returns SMX_ERR_INVALID_ARGUMENT if
 * anything was found. Only the given arrays are read. */
int smx_validate_inputs(smx_handle h, int feature_rows, long* counts, long* total);

/* Energy + virial reduction for callers that cannot let the library allocate device memory: hosts
 * that give the whole GPU to their own memory pool at start-up, jobs with a fixed device-memory
 * budget, and step loops that cannot take the device-wide synchronisation of cudaMalloc / cudaFree.
 * This entry point has no counterpart in the reference (its callers reduce on the host,
 * pair_symmetrix_mace.cpp:324-368). It computes what smx_reduce_forces returns as `energy` and
 * `virial` -- out7 = {sum of node_energies, virial xx, yy, zz, xy, xz, yz} -- from device arrays the
 * caller passes (node_energies[num_nodes], xyz[3*num_edges], node_forces[3*num_edges], out7[7], all
 * device pointers on the current GPU), asynchronously on `stream` (a cudaStream_t, may be NULL).
 * It calls no cudaMalloc, cudaFree or allocating library routine: its scratch is a 229,376-byte
 * array compiled into the library and resident on every GPU that loads it. Limits: at most
 * 16,777,216 edges and as many nodes; larger inputs return SMX_ERR_INVALID_ARGUMENT with a message
 * in `errbuf` (capacity `errbuf_len`, may be NULL). All calls on one GPU share the scratch array,
 * which keeps the previous call's contents: calls whose kernels overlap on the device race. The first
 * call on each GPU looks up the array's device address (and, with CUDA's lazy loading, may make the
 * driver load the library's kernels, which is the driver's own allocation); make it before any
 * stream capture starts. */
int smx_energy_virial_noalloc(const double* node_energies, int num_nodes, const double* xyz,
                              const double* node_forces, long num_edges, double* out7, void* stream,
                              char* errbuf, int errbuf_len);

#ifdef __cplusplus
}
#endif
#endif /* SYMMETRIX_B200_H */
