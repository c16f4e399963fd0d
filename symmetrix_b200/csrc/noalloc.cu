// Energy + virial reduction that allocates nothing.
//
// Some hosts of this library cannot let it allocate device memory while they run: a molecular-
// dynamics code that hands the whole GPU to its own memory pool at start-up has nothing left for
// a cudaMalloc in the middle of a time step, and a job that shares a GPU under a fixed memory
// budget must know every byte in advance. cudaMalloc / cudaFree also synchronise the whole device,
// which a step loop that overlaps work on several streams cannot afford. For such callers this
// file offers the caller-side reduction of per-edge partial forces (total energy and the six
// virial components) as one call whose only scratch is a fixed array compiled into the library.
//
// The scratch is the file-scope array `g_partials` below: 4096 rows of 7 doubles = 229,376 bytes,
// resident on every GPU that loads the library until the process exits. Each CUDA block reduces a
// fixed chunk of 4096 items into one row, so the call handles at most 4096 * 4096 = 16,777,216
// edges (and as many nodes); larger inputs are rejected. Every launched block overwrites its whole
// row and the final pass reads only the rows of the current call, so nothing has to be cleared
// between calls. All calls on one GPU share the array: two calls whose kernels overlap on the
// device (different streams, or different host threads) race on it and give wrong sums.
//
// The device address of the array is looked up once per GPU with cudaGetSymbolAddress (the name
// `g_partials` itself is only a host-side stand-in in host code, never a device pointer) by the
// first call made while that GPU is current; make that first call before starting any stream
// capture.
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "../../include/symmetrix_b200.h"

namespace {

constexpr int kThreads = 256;
constexpr int kItemsPerThread = 16;
constexpr int kChunk = kThreads * kItemsPerThread;        // 4096 items per block
constexpr int kMaxBlocks = 4096;                          // rows of scratch
constexpr long kMaxItems = static_cast<long>(kMaxBlocks) * kChunk;   // 16,777,216
constexpr int kMaxDevices = 64;

static __device__ __align__(256) double g_partials[kMaxBlocks * 7];

// Block b reduces items [b * kChunk, (b + 1) * kChunk) of the node energies and of the edge list
// into row b: {energy, xx, yy, zz, xy, xz, yz}; virial convention of
// pair_symmetrix/pair_symmetrix_mace.cpp:349-368.
__global__ void __launch_bounds__(kThreads) chunk_partials_kernel(int num_nodes, long num_edges, const double* __restrict__ node_energies,
                                                                  const double* __restrict__ xyz, const double* __restrict__ nf,
                                                                  double* __restrict__ partials) {
    __shared__ double sh[7][kThreads];
    double v[7] = {0, 0, 0, 0, 0, 0, 0};
    const long base = static_cast<long>(blockIdx.x) * kChunk;
    for (int it = 0; it < kItemsPerThread; ++it) {
        const long idx = base + static_cast<long>(it) * kThreads + threadIdx.x;
        if (idx < num_nodes) v[0] += node_energies[idx];
        if (idx < num_edges) {
            const double x = xyz[3 * idx], y = xyz[3 * idx + 1], z = xyz[3 * idx + 2];
            const double fx = nf[3 * idx], fy = nf[3 * idx + 1], fz = nf[3 * idx + 2];
            v[1] += x * fx; v[2] += y * fy; v[3] += z * fz;
            v[4] += 0.5 * (x * fy + y * fx); v[5] += 0.5 * (x * fz + z * fx); v[6] += 0.5 * (y * fz + z * fy);
        }
    }
    for (int c = 0; c < 7; ++c) sh[c][threadIdx.x] = v[c];
    __syncthreads();
    for (int s = kThreads >> 1; s > 0; s >>= 1) {
        if (threadIdx.x < s)
            for (int c = 0; c < 7; ++c) sh[c][threadIdx.x] += sh[c][threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x < 7) partials[blockIdx.x * 7 + threadIdx.x] = sh[threadIdx.x][0];
}

// One warp per component (7 warps): lane l adds the rows l, l + 32, ... in order, then a fixed shuffle tree combines the lanes.
__global__ void sum_rows_kernel(int num_rows, const double* __restrict__ partials, double* __restrict__ out7) {
    const int comp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (comp >= 7) return;
    double s = 0;
    for (int b = lane; b < num_rows; b += 32) s += partials[b * 7 + comp];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_down_sync(0xffffffffu, s, off);
    if (lane == 0) out7[comp] = s;
}

std::mutex g_setup_mutex;
double* g_scratch_of_device[kMaxDevices] = {};

int fail(int status, char* errbuf, int errbuf_len, const char* what, const char* detail = "") {
    if (errbuf && errbuf_len > 0) std::snprintf(errbuf, static_cast<size_t>(errbuf_len), "%s%s", what, detail);
    return status;
}

}  // namespace

extern "C" int smx_energy_virial_noalloc(const double* node_energies, int num_nodes, const double* xyz, const double* node_forces,
                                         long num_edges, double* out7, void* stream, char* errbuf, int errbuf_len) {
    if (num_nodes < 0 || num_edges < 0) return fail(SMX_ERR_INVALID_ARGUMENT, errbuf, errbuf_len, "smx_energy_virial_noalloc: negative size");
    if (num_nodes > kMaxItems || num_edges > kMaxItems)
        return fail(SMX_ERR_INVALID_ARGUMENT, errbuf, errbuf_len,
                    "smx_energy_virial_noalloc: input exceeds the fixed scratch capacity of 16777216 edges / nodes; "
                    "use smx_reduce_forces, which allocates");
    if (!out7 || (num_nodes > 0 && !node_energies) || (num_edges > 0 && (!xyz || !node_forces)))
        return fail(SMX_ERR_INVALID_ARGUMENT, errbuf, errbuf_len, "smx_energy_virial_noalloc: null pointer");
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return fail(SMX_ERR_CUDA, errbuf, errbuf_len, "cudaGetDevice: ", cudaGetErrorString(err));
    if (dev < 0 || dev >= kMaxDevices) return fail(SMX_ERR_INVALID_ARGUMENT, errbuf, errbuf_len, "smx_energy_virial_noalloc: device ordinal beyond 63");
    double* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        if (!g_scratch_of_device[dev]) {
            // one-time set-up for this GPU: resolve the device address of the static array
            double* p = nullptr;
            err = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_partials);
            if (err != cudaSuccess || !p) return fail(SMX_ERR_CUDA, errbuf, errbuf_len, "cudaGetSymbolAddress: ", cudaGetErrorString(err));
            g_scratch_of_device[dev] = p;
        }
        scratch = g_scratch_of_device[dev];
    }
    const long items = num_nodes > num_edges ? num_nodes : num_edges;
    const int blocks = static_cast<int>((items + kChunk - 1) / kChunk);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (blocks > 0) chunk_partials_kernel<<<blocks, kThreads, 0, s>>>(num_nodes, num_edges, node_energies, xyz, node_forces, scratch);
    sum_rows_kernel<<<1, 7 * 32, 0, s>>>(blocks, scratch, out7);
    err = cudaGetLastError();
    if (err != cudaSuccess) return fail(SMX_ERR_CUDA, errbuf, errbuf_len, "kernel launch: ", cudaGetErrorString(err));
    return SMX_OK;
}
