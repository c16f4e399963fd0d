// Full periodic neighbour list on the device, written directly in the evaluator's CSR form.
//
// Edge rule (identical, operation for operation, to symmetrix_b200/structures.py::neighbor_list,
// which restates what the reference's callers do, pair_symmetrix/pair_symmetrix_mace.cpp:249-315):
//   p = x_j + ((n0*a0 + n1*a1) + n2*a2)        image position, float64, no fused multiply-add
//   d = p - x_i
//   keep iff (d0*d0 + d1*d1) + d2*d2 < r_cut*r_cut, excluding i == j with a zero shift
// Rows are ordered by (sender index, shift code), so the list is a pure function of its inputs. One warp builds one row.
// Candidates come from a uniform grid over fractional coordinates whose cells are at least
// r_cut(1+1e-9) thick. Positions need not lie inside the cell: along a periodic axis an atom is binned by its
// wrapped fractional coordinate, and the whole cell vectors w_i it is away from the cell are folded into the
// integer shift of its edges (n = n' + w_i - w_j for the image n' found between the wrapped positions), so xyz
// is still formed from the positions as given. Along a non-periodic axis outliers go to the edge bins.
#pragma once

#include <cuda_runtime.h>

#include <cmath>

#include <cub/cub.cuh>

#include "common.cuh"

namespace smx {

struct NeighGrid {
    double cell[9];      // rows are lattice vectors
    double inv[9];       // inverse of the cell matrix: frac = pos . inv
    int nb[3];           // bins per axis
    int reach[3];        // bins to search on each side
    int pbc[3];
    double rc2;
};

// Bin of an atom and (w3) the whole cell vectors its position is away from the cell along the periodic axes.
__device__ __forceinline__ int neigh_bin(const NeighGrid& g, const double* x, int* b3, int* w3) {
    int id = 0;
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        double s = x[0] * g.inv[0 * 3 + a] + x[1] * g.inv[1 * 3 + a] + x[2] * g.inv[2 * 3 + a];
        const double wf = g.pbc[a] ? floor(s) : 0.0;
        // far outliers are clamped here and rejected by the shift-range check of neigh_rows_kernel
        w3[a] = static_cast<int>(wf < -1e6 ? -1e6 : (wf > 1e6 ? 1e6 : wf));
        s -= wf;
        int b = static_cast<int>(floor(s * g.nb[a]));
        b = b < 0 ? 0 : (b >= g.nb[a] ? g.nb[a] - 1 : b);
        b3[a] = b;
        id = id * g.nb[a] + b;
    }
    return id;
}

static __global__ void neigh_bin_kernel(int n, const double* __restrict__ pos, NeighGrid g, int* __restrict__ bin_of,
                                        int* __restrict__ wrap) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        int b3[3];
        bin_of[i] = neigh_bin(g, pos + 3 * i, b3, wrap + 3 * i);
    }
}

// Exact edge test; returns true and fills d/r2 when image (j, n) of atom j is a neighbour of i.
__device__ __forceinline__ bool neigh_test(const NeighGrid& g, const double* xi, const double* xj, int n0, int n1, int n2,
                                           double* d, double* r2) {
#pragma unroll
    for (int c = 0; c < 3; ++c) {
        const double sv = __dadd_rn(__dadd_rn(__dmul_rn(double(n0), g.cell[0 + c]), __dmul_rn(double(n1), g.cell[3 + c])),
                                    __dmul_rn(double(n2), g.cell[6 + c]));
        const double p = __dadd_rn(xj[c], sv);
        d[c] = __dsub_rn(p, xi[c]);
    }
    *r2 = __dadd_rn(__dadd_rn(__dmul_rn(d[0], d[0]), __dmul_rn(d[1], d[1])), __dmul_rn(d[2], d[2]));
    return *r2 < g.rc2;
}

// Sort key of an edge inside its row: sender first, then the shift in lexicographic order. Shifts are kept in
// 10 bits per axis (|n| <= kNeighMaxShift).
constexpr int kNeighMaxShift = 511;
__device__ __forceinline__ unsigned long long neigh_key(int j, int n0, int n1, int n2) {
    const unsigned long long code = (static_cast<unsigned long long>(n0 + 512) * 1024 + (n1 + 512)) * 1024 + (n2 + 512);
    return (static_cast<unsigned long long>(j) << 32) | code;
}

// One warp per receiver atom; the lanes share the candidates of the 27 (or more) bins around the atom's bin.
// COUNT: number of edges of the row. Otherwise: the keys of the row are collected in shared memory in traversal order,
// ranked (keys are unique, so the rank of a key is the number of smaller keys: the row comes out ordered by
// (sender, shift) whatever the traversal order was), and each key is expanded into the edge arrays with the same
// arithmetic that tested it. Rows longer than kNeighRowCap keys are ranked in global memory by the same rule.
constexpr int kNeighWarps = 4;           // warps per CTA
constexpr int kNeighRowCap = 512;        // keys of one row held in shared memory

template <bool COUNT>
static __global__ void __launch_bounds__(kNeighWarps * 32) neigh_rows_kernel(
    int n, const double* __restrict__ pos, const int* __restrict__ types, NeighGrid g, const int* __restrict__ bin_start,
    const int* __restrict__ sorted_atoms, const int* __restrict__ wrap, int* __restrict__ shift_overflow, int* __restrict__ num_neigh,
    const long long* __restrict__ first_neigh, unsigned long long* __restrict__ keys, int* __restrict__ neigh_indices,
    int* __restrict__ neigh_types, int* __restrict__ shifts, double* __restrict__ xyz, double* __restrict__ r) {
    __shared__ unsigned long long row_keys[COUNT ? 1 : kNeighWarps][COUNT ? 1 : kNeighRowCap];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps_total = gridDim.x * kNeighWarps;
    for (int i = blockIdx.x * kNeighWarps + warp; i < n; i += warps_total) {
        const double xi[3] = {pos[3 * i], pos[3 * i + 1], pos[3 * i + 2]};
        int b3[3], wi[3];
        neigh_bin(g, xi, b3, wi);
        const long long row_begin = COUNT ? 0 : first_neigh[i];
        int count = 0;                     // edges found so far (the same value in every lane)
        for (int o0 = -g.reach[0]; o0 <= g.reach[0]; ++o0) {
            const int v0 = b3[0] + o0;
            const int n0 = static_cast<int>(floor(double(v0) / g.nb[0]));
            if (n0 != 0 && !g.pbc[0]) continue;
            const int c0 = v0 - n0 * g.nb[0];
            for (int o1 = -g.reach[1]; o1 <= g.reach[1]; ++o1) {
                const int v1 = b3[1] + o1;
                const int n1 = static_cast<int>(floor(double(v1) / g.nb[1]));
                if (n1 != 0 && !g.pbc[1]) continue;
                const int c1 = v1 - n1 * g.nb[1];
                for (int o2 = -g.reach[2]; o2 <= g.reach[2]; ++o2) {
                    const int v2 = b3[2] + o2;
                    const int n2 = static_cast<int>(floor(double(v2) / g.nb[2]));
                    if (n2 != 0 && !g.pbc[2]) continue;
                    const int c2 = v2 - n2 * g.nb[2];
                    const int bin = (c0 * g.nb[1] + c1) * g.nb[2] + c2;
                    const int s_end = bin_start[bin + 1];
                    for (int s0 = bin_start[bin]; s0 < s_end; s0 += 32) {
                        const int s = s0 + lane;
                        bool hit = false;
                        unsigned long long key = 0;
                        if (s < s_end) {
                            const int j = sorted_atoms[s];
                            if (!(j == i && n0 == 0 && n1 == 0 && n2 == 0)) {
                                // shift between the positions as given: image between the wrapped positions + the two wraps
                                const int m0 = n0 + wi[0] - wrap[3 * j], m1 = n1 + wi[1] - wrap[3 * j + 1], m2 = n2 + wi[2] - wrap[3 * j + 2];
                                double d[3], r2;
                                if (neigh_test(g, xi, pos + 3 * j, m0, m1, m2, d, &r2)) {
                                    hit = true;
                                    if (COUNT && (abs(m0) > kNeighMaxShift || abs(m1) > kNeighMaxShift || abs(m2) > kNeighMaxShift)) *shift_overflow = 1;
                                    key = neigh_key(j, m0, m1, m2);
                                }
                            }
                        }
                        const unsigned mask = __ballot_sync(0xffffffffu, hit);
                        if (!COUNT && hit) {
                            const int slot = count + __popc(mask & ((1u << lane) - 1u));
                            if (slot < kNeighRowCap) row_keys[warp][slot] = key;
                            keys[row_begin + slot] = key;         // long rows are ranked from here
                        }
                        count += __popc(mask);
                    }
                }
            }
        }
        if (COUNT) {
            if (lane == 0) num_neigh[i] = count;
            continue;
        }
        __syncwarp();
        const bool in_smem = count <= kNeighRowCap;
        for (int a = lane; a < count; a += 32) {
            const unsigned long long key = in_smem ? row_keys[warp][a] : keys[row_begin + a];
            int rank = 0;
            for (int b = 0; b < count; ++b) rank += (in_smem ? row_keys[warp][b] : keys[row_begin + b]) < key ? 1 : 0;
            const long long e = row_begin + rank;
            const int j = static_cast<int>(key >> 32);
            const unsigned int code = static_cast<unsigned int>(key & 0xffffffffu);
            const int n2 = static_cast<int>(code % 1024) - 512, n1 = static_cast<int>((code / 1024) % 1024) - 512,
                      n0 = static_cast<int>(code / (1024 * 1024)) - 512;
            double d[3], r2;
            neigh_test(g, xi, pos + 3 * j, n0, n1, n2, d, &r2);
            neigh_indices[e] = j;
            neigh_types[e] = types[j];
            shifts[3 * e] = n0; shifts[3 * e + 1] = n1; shifts[3 * e + 2] = n2;
            xyz[3 * e] = d[0]; xyz[3 * e + 1] = d[1]; xyz[3 * e + 2] = d[2];
            r[e] = __dsqrt_rn(r2);
        }
        __syncwarp();
    }
}

static __global__ void neigh_iota_kernel(int n, int* out) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) out[i] = i;
}
static __global__ void neigh_offsets_kernel(int n, const int* __restrict__ sorted_keys, int num_values, int* __restrict__ offsets) {
    for (int v = blockIdx.x * blockDim.x + threadIdx.x; v <= num_values; v += gridDim.x * blockDim.x) {
        int lo = 0, hi = n;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (sorted_keys[mid] < v) lo = mid + 1; else hi = mid;
        }
        offsets[v] = lo;
    }
}

struct NeighCast {
    __host__ __device__ long long operator()(const int& v) const { return static_cast<long long>(v); }
};

class NeighborBuilder {
public:
    DevBuf<double> d_pos;
    DevBuf<int> bin_of, sorted_bins, sorted_atoms, iota, bin_start, wrap, overflow;
    DevBuf<long long> first;
    DevBuf<unsigned long long> keys;
    DevBuf<unsigned char> tmp;

    void build(int n, const double* pos, const int* d_types, const double* cell, const int* pbc, double r_cut, bool pos_on_device,
               cudaStream_t stream, long& launches, DevBuf<int>& num_neigh, DevBuf<int>& neigh_indices, DevBuf<int>& neigh_types,
               DevBuf<int>& shifts, DevBuf<double>& xyz, DevBuf<double>& r, long& num_edges) {
        if (!(r_cut > 0.0)) throw ArgError("build_neighbors: r_cut must be positive");
        NeighGrid g{};
        for (int q = 0; q < 9; ++q) g.cell[q] = cell[q];
        const double* a = cell;
        const double det = a[0] * (a[4] * a[8] - a[5] * a[7]) - a[1] * (a[3] * a[8] - a[5] * a[6]) + a[2] * (a[3] * a[7] - a[4] * a[6]);
        if (std::fabs(det) < 1e-300) throw ArgError("build_neighbors: singular cell");
        g.inv[0] = (a[4] * a[8] - a[5] * a[7]) / det; g.inv[1] = (a[2] * a[7] - a[1] * a[8]) / det; g.inv[2] = (a[1] * a[5] - a[2] * a[4]) / det;
        g.inv[3] = (a[5] * a[6] - a[3] * a[8]) / det; g.inv[4] = (a[0] * a[8] - a[2] * a[6]) / det; g.inv[5] = (a[2] * a[3] - a[0] * a[5]) / det;
        g.inv[6] = (a[3] * a[7] - a[4] * a[6]) / det; g.inv[7] = (a[1] * a[6] - a[0] * a[7]) / det; g.inv[8] = (a[0] * a[4] - a[1] * a[3]) / det;
        long long total_bins = 1;
        for (int ax = 0; ax < 3; ++ax) {
            const double* u = cell + 3 * ((ax + 1) % 3);
            const double* v = cell + 3 * ((ax + 2) % 3);
            const double cx = u[1] * v[2] - u[2] * v[1], cy = u[2] * v[0] - u[0] * v[2], cz = u[0] * v[1] - u[1] * v[0];
            const double height = std::fabs(det) / std::sqrt(cx * cx + cy * cy + cz * cz);
            const double rc = r_cut * (1.0 + 1e-9);
            int nbins = static_cast<int>(std::floor(height / rc));
            if (nbins < 1) nbins = 1;
            if (nbins > 256) nbins = 256;
            g.nb[ax] = nbins;
            g.reach[ax] = static_cast<int>(std::ceil(rc / (height / nbins)));
            if (!pbc[ax] && g.reach[ax] > nbins) g.reach[ax] = nbins;
            if (g.reach[ax] > 63 * nbins) throw ArgError("build_neighbors: cell far smaller than r_cut");
            g.pbc[ax] = pbc[ax] ? 1 : 0;
            total_bins *= nbins;
        }
        g.rc2 = r_cut * r_cut;
        const double* dpos = pos;
        if (!pos_on_device) {
            d_pos.resize(3 * static_cast<size_t>(n), stream);
            if (n) SMX_CUDA(cudaMemcpyAsync(d_pos.p, pos, 3 * static_cast<size_t>(n) * sizeof(double), cudaMemcpyHostToDevice, stream));
            dpos = d_pos.p;
        }
        num_neigh.resize(n, stream);
        num_edges = 0;
        if (n == 0) {
            neigh_indices.resize(0, stream); neigh_types.resize(0, stream); shifts.resize(0, stream); xyz.resize(0, stream); r.resize(0, stream);
            return;
        }
        const int nbins = static_cast<int>(total_bins);
        const int blocks = std::min(4096, (n + 127) / 128);
        bin_of.resize(n, stream); sorted_bins.resize(n, stream); sorted_atoms.resize(n, stream); iota.resize(n, stream);
        bin_start.resize(static_cast<size_t>(nbins) + 1, stream);
        wrap.resize(3 * static_cast<size_t>(n), stream);
        overflow.resize(1, stream);
        overflow.zero(stream);
        neigh_bin_kernel<<<blocks, 128, 0, stream>>>(n, dpos, g, bin_of.p, wrap.p);
        neigh_iota_kernel<<<blocks, 128, 0, stream>>>(n, iota.p);
        launches += 2;
        int bits = 1;
        while ((1LL << bits) < total_bins) ++bits;
        size_t bytes = 0;
        SMX_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, bytes, bin_of.p, sorted_bins.p, iota.p, sorted_atoms.p, n, 0, bits, stream));
        tmp.resize(bytes, stream);
        SMX_CUDA(cub::DeviceRadixSort::SortPairs(tmp.p, bytes, bin_of.p, sorted_bins.p, iota.p, sorted_atoms.p, n, 0, bits, stream));
        neigh_offsets_kernel<<<std::min(1024, (nbins + 128) / 128), 128, 0, stream>>>(n, sorted_bins.p, nbins, bin_start.p);
        launches += 2;
        const int row_blocks = std::min(16384, (n + kNeighWarps - 1) / kNeighWarps);      // one warp per atom
        neigh_rows_kernel<true><<<row_blocks, kNeighWarps * 32, 0, stream>>>(n, dpos, d_types, g, bin_start.p, sorted_atoms.p, wrap.p, overflow.p, num_neigh.p, nullptr, nullptr,
                                                          nullptr, nullptr, nullptr, nullptr, nullptr);
        launches += 1;
        first.resize(static_cast<size_t>(n) + 1, stream);
        cub::TransformInputIterator<long long, NeighCast, const int*> it(num_neigh.p, NeighCast());
        SMX_CUDA(cub::DeviceScan::ExclusiveSum(nullptr, bytes, it, first.p, n, stream));
        tmp.resize(bytes, stream);
        SMX_CUDA(cub::DeviceScan::ExclusiveSum(tmp.p, bytes, it, first.p, n, stream));
        launches += 1;
        long long last_first = 0;
        int last_count = 0, shift_overflow = 0;
        SMX_CUDA(cudaMemcpyAsync(&shift_overflow, overflow.p, sizeof(int), cudaMemcpyDeviceToHost, stream));
        SMX_CUDA(cudaMemcpyAsync(&last_first, first.p + (n - 1), sizeof(long long), cudaMemcpyDeviceToHost, stream));
        SMX_CUDA(cudaMemcpyAsync(&last_count, num_neigh.p + (n - 1), sizeof(int), cudaMemcpyDeviceToHost, stream));
        SMX_CUDA(cudaStreamSynchronize(stream));
        if (shift_overflow) throw ArgError("build_neighbors: an atom lies more than 500 cell lengths outside the cell along a periodic axis");
        const long long total = last_first + last_count;
        num_edges = static_cast<long>(total);
        keys.resize(total, stream);
        neigh_indices.resize(total, stream); neigh_types.resize(total, stream); shifts.resize(3 * total, stream);
        xyz.resize(3 * total, stream); r.resize(total, stream);
        if (total > 0) {
            neigh_rows_kernel<false><<<row_blocks, kNeighWarps * 32, 0, stream>>>(n, dpos, d_types, g, bin_start.p, sorted_atoms.p, wrap.p, overflow.p, nullptr, first.p, keys.p,
                                                               neigh_indices.p, neigh_types.p, shifts.p, xyz.p, r.p);
            launches += 1;
        }
        cudaError_t err = cudaGetLastError();
        if (err != cudaSuccess) throw CudaError(std::string("neighbour list: ") + cudaGetErrorString(err));
    }
};

}  // namespace smx
