// CUDA kernels of the MACE energy+force path for sm_100a.
//
// Data layout in HBM (all row-major, channel index fastest, one arithmetic type T per evaluator):
//   node features  A0/A1 [N][16][K], M0/H1 [rows][nLM][K], Phi1 [N][Q][K], M1/H2 [N][K]
//   spline tables  [pair][bin][function block][K][4] in float, [pair][bin][function block][2][K][2] in double
//                  (16-byte vector loads that a warp issues over contiguous 512-byte spans)
//   contraction    coefficients [element][monomial][K]
// One thread owns one channel k of one receiver node, so every global access is a contiguous
// run of K values across the CTA. Per-edge quantities that do not depend on the channel
// (harmonics, their gradients, coupling blocks, spline bin) are computed once per edge into
// shared memory and broadcast. No per-edge channel array (R0, R1, Y, Phi1r of the reference,
// libsymmetrix/source/mace.hpp:44-113) is ever written to HBM.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include <utility>

#include "tp_tables.hpp"
#include "generated/poly_canon.hpp"

namespace smx {

#ifndef SMX_EDGE_BATCH
#define SMX_EDGE_BATCH 32
#endif
constexpr int kEdgeBatch = SMX_EDGE_BATCH;   // edges staged in shared memory per pass (one staging latency and two barriers per batch)
// thread t of a CTA stages edge t of a batch and a CTA may be a single warp, so a batch holds at most 32 edges (the 40-edge
// measurement was a build for 128-channel models only, with this check lifted)
#ifndef SMX_EDGE_BATCH_UNCHECKED
static_assert(kEdgeBatch >= 1 && kEdgeBatch <= 32, "SMX_EDGE_BATCH must be between 1 and 32");
#endif
constexpr int kChannelBlock = 128;  // threads per CTA of the edge kernels; more channels are done in chunks
constexpr int kMaxWarps = kChannelBlock / 32;

// Compile-time loop: f(std::integral_constant<int, 0>{}), ..., f(std::integral_constant<int, N-1>{}).
// The tensor-product kernels index their register accumulators with path-dependent offsets, which
// must be constants for the accumulators to stay in registers.
template <typename F, int... I>
__device__ __forceinline__ void static_for_impl(F&& f, std::integer_sequence<int, I...>) {
    (f(std::integral_constant<int, I>{}), ...);
}
template <int N, typename F>
__device__ __forceinline__ void static_for(F&& f) {
    static_for_impl(f, std::make_integer_sequence<int, N>{});
}
template <int LF>
struct TPConst {
    static constexpr TPTable t = make_tp_table(LF);
};

template <typename T> struct Vec4;
template <> struct alignas(16) Vec4<float> { float x, y, z, w; };
template <> struct alignas(32) Vec4<double> { double x, y, z, w; };

// The four cubic coefficients of channel k from one (pair, bin, function-block) row of 4*K values.
// float rows are [K][4]: one 16-byte load per thread, a warp reads 512 contiguous bytes.
// double rows are [2][K][2] (c0,c1 of every channel, then c2,c3 of every channel): each of the two 16-byte
// loads of a warp is again 512 contiguous bytes, i.e. 4 L1 wavefronts instead of the 8 an interleaved
// [K][4] row of doubles (32-byte stride between lanes) costs.
template <typename T>
__device__ __forceinline__ Vec4<T> load_coef(const T* row, int k, int K);
template <>
__device__ __forceinline__ Vec4<float> load_coef<float>(const float* row, int k, int) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(row) + k);
    return {v.x, v.y, v.z, v.w};
}
template <>
__device__ __forceinline__ Vec4<double> load_coef<double>(const double* row, int k, int K) {
    const double2 a = __ldg(reinterpret_cast<const double2*>(row) + k);
    const double2 b = __ldg(reinterpret_cast<const double2*>(row) + K + k);
    return {a.x, a.y, b.x, b.y};
}

// ---------------------------------------------------------------------------------------------
// Bulk asynchronous copies (TMA, cp.async.bulk) of spline rows into shared memory, completed on an
// mbarrier. Every wait is bounded: a wait that runs out returns false and the caller records it.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("{\n\t.reg .b64 t;\n\tmbarrier.arrive.shared::cta.b64 t, [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("{\n\t.reg .b64 t;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 t, [%0], %1;\n\t}" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
constexpr unsigned kMbarSpinLimit = 1u << 22;
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, unsigned limit = kMbarSpinLimit) {
    const uint32_t addr = smem_u32(bar);
    for (unsigned spin = 0; spin < limit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
// global -> shared, both addresses 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// Channel `kl` of a staged row chunk of `Kc` channels: same layouts as load_coef with K = Kc.
template <typename T>
__device__ __forceinline__ Vec4<T> lds_coef(const T* slot, int p, int kl, int Kc);
template <>
__device__ __forceinline__ Vec4<float> lds_coef<float>(const float* slot, int p, int kl, int Kc) {
    const float4 v = reinterpret_cast<const float4*>(slot)[p * Kc + kl];
    return {v.x, v.y, v.z, v.w};
}
template <>
__device__ __forceinline__ Vec4<double> lds_coef<double>(const double* slot, int p, int kl, int Kc) {
    const double2 a = reinterpret_cast<const double2*>(slot)[(2 * p) * Kc + kl];
    const double2 b = reinterpret_cast<const double2*>(slot)[(2 * p + 1) * Kc + kl];
    return {a.x, a.y, b.x, b.y};
}

// One thread: start the copy of the chunk [kc, kc + Kc) of all P function blocks of a spline row into a slot.
template <typename T>
__device__ __forceinline__ void issue_row_copy(T* slot, const T* row, int P, int K, int kc, int Kc, unsigned long long* bar) {
    const unsigned bytes = 4u * P * Kc * sizeof(T);
    mbar_expect_tx(bar, bytes);
    if (Kc == K) {
        bulk_copy_g2s(slot, row, bytes, bar);
    } else if constexpr (sizeof(T) == 4) {
        for (int p = 0; p < P; ++p) bulk_copy_g2s(slot + 4 * p * Kc, row + 4 * (p * K + kc), 16u * Kc, bar);
    } else {
        for (int q = 0; q < 2 * P; ++q) bulk_copy_g2s(slot + 2 * q * Kc, row + 2 * (q * K + kc), 16u * Kc, bar);
    }
}

template <typename T>
__device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sum each of 16 per-lane values over the warp with 16 shuffles instead of 80: every step halves the
// number of values a lane carries by exchanging the other half with its partner. On return the lane
// holds the warp-wide sum of value `index` (lanes that differ only in bit 0 hold the same value).
template <typename T>
__device__ __forceinline__ T warp_reduce_scatter16(const T (&v)[16], int lane, int& index) {
    const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4, b1 = lane & 2;
    T w8[8], w4[4], w2[2];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const T send = b4 ? v[i] : v[i + 8], keep = b4 ? v[i + 8] : v[i];
        w8[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const T send = b3 ? w8[i] : w8[i + 4], keep = b3 ? w8[i + 4] : w8[i];
        w4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const T send = b2 ? w4[i] : w4[i + 2], keep = b2 ? w4[i + 2] : w4[i];
        w2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    }
    const T send = b1 ? w2[0] : w2[1], keep = b1 ? w2[1] : w2[0];
    T w1 = keep + __shfl_xor_sync(0xffffffffu, send, 2);
    w1 += __shfl_xor_sync(0xffffffffu, w1, 1);
    index = (b4 ? 8 : 0) + (b3 ? 4 : 0) + (b2 ? 2 : 0) + (b1 ? 1 : 0);
    return w1;
}

// Per-edge partial force from the warp-reduced adjoints, written by one thread per edge:
//   nf -= xhat * dE/dr + sum_lm dE/dY_lm * grad Y_lm
// red[w][e][0..15] = dE/dY_lm summed over the channels of warp w, red[w][e][16] = dE/dr.
template <typename T, int EB>
__device__ __forceinline__ void finish_edge_force(const T (*red)[EB][17], int nwarps, int e, const T* dY0, const T* dY1, const T* dY2,
                                                  T ux, T uy, T uz, double* nf) {
    double tr = 0, fx = 0, fy = 0, fz = 0;
    for (int w = 0; w < nwarps; ++w) tr += red[w][e][16];
#pragma unroll
    for (int lm = 0; lm < kNumLm; ++lm) {
        double wv = 0;
        for (int w = 0; w < nwarps; ++w) wv += red[w][e][lm];
        fx += wv * double(dY0[lm]); fy += wv * double(dY1[lm]); fz += wv * double(dY2[lm]);
    }
    nf[0] -= double(ux) * tr + fx;
    nf[1] -= double(uy) * tr + fy;
    nf[2] -= double(uz) * tr + fz;
}

// ---------------------------------------------------------------------------------------------
// Real spherical harmonics up to l = 3 of the direction (a, b, c) = xyz / r, in the convention the
// reference feeds its tensor products with (mace.cpp:118-148: orthonormal real harmonics of the
// axis-shuffled vector (z, x, y), times 2 sqrt(pi), lm = l*l + l + m), written as polynomials in
// the un-shuffled components. g[c][lm] receives the Cartesian gradient d Y_lm / d xyz_c.
// ---------------------------------------------------------------------------------------------
template <typename T, bool GRAD>
__host__ __device__ inline void real_sh3(T a, T b, T c, T inv_r, T* __restrict__ Y, T (*__restrict__ g)[kNumLm]) {
    const T s3 = T(1.7320508075688772935), s15 = T(3.8729833462074168852), s5h = T(1.1180339887498948482);
    const T s105 = T(10.246950765959598383), s7h = T(1.3228756555322952953);
    const T k9 = T(2.0916500663351888699);   // sqrt(35/8)
    const T k11 = T(1.6201851746019651311);  // sqrt(21/8)
    const T aa = a * a, bb = b * b, cc = c * c;
    Y[0] = T(1);
    Y[1] = s3 * a; Y[2] = s3 * b; Y[3] = s3 * c;
    Y[4] = s15 * c * a;
    Y[5] = s15 * a * b;
    Y[6] = s5h * (T(3) * bb - T(1));
    Y[7] = s15 * c * b;
    Y[8] = T(0.5) * s15 * (cc - aa);
    Y[9] = k9 * a * (T(3) * cc - aa);
    Y[10] = s105 * a * b * c;
    Y[11] = k11 * a * (T(5) * bb - T(1));
    Y[12] = s7h * b * (T(5) * bb - T(3));
    Y[13] = k11 * c * (T(5) * bb - T(1));
    Y[14] = T(0.5) * s105 * b * (cc - aa);
    Y[15] = k9 * c * (cc - T(3) * aa);
    if constexpr (GRAD) {
        T d[3][kNumLm];
        d[0][0] = 0; d[1][0] = 0; d[2][0] = 0;
        d[0][1] = s3; d[1][1] = 0; d[2][1] = 0;
        d[0][2] = 0; d[1][2] = s3; d[2][2] = 0;
        d[0][3] = 0; d[1][3] = 0; d[2][3] = s3;
        d[0][4] = s15 * c; d[1][4] = 0; d[2][4] = s15 * a;
        d[0][5] = s15 * b; d[1][5] = s15 * a; d[2][5] = 0;
        d[0][6] = 0; d[1][6] = T(6) * s5h * b; d[2][6] = 0;
        d[0][7] = 0; d[1][7] = s15 * c; d[2][7] = s15 * b;
        d[0][8] = -s15 * a; d[1][8] = 0; d[2][8] = s15 * c;
        d[0][9] = k9 * T(3) * (cc - aa); d[1][9] = 0; d[2][9] = k9 * T(6) * a * c;
        d[0][10] = s105 * b * c; d[1][10] = s105 * a * c; d[2][10] = s105 * a * b;
        d[0][11] = k11 * (T(5) * bb - T(1)); d[1][11] = k11 * T(10) * a * b; d[2][11] = 0;
        d[0][12] = 0; d[1][12] = s7h * (T(15) * bb - T(3)); d[2][12] = 0;
        d[0][13] = 0; d[1][13] = k11 * T(10) * b * c; d[2][13] = k11 * (T(5) * bb - T(1));
        d[0][14] = -s105 * a * b; d[1][14] = T(0.5) * s105 * (cc - aa); d[2][14] = s105 * b * c;
        d[0][15] = -k9 * T(6) * a * c; d[1][15] = 0; d[2][15] = k9 * T(3) * (cc - aa);
        // chain rule through u = xyz / r: grad = (d - u (u . d)) / r
#pragma unroll
        for (int lm = 0; lm < kNumLm; ++lm) {
            const T rad = d[0][lm] * a + d[1][lm] * b + d[2][lm] * c;
            g[0][lm] = (d[0][lm] - rad * a) * inv_r;
            g[1][lm] = (d[1][lm] - rad * b) * inv_r;
            g[2][lm] = (d[2][lm] - rad * c) * inv_r;
        }
    }
}

// Per-edge, channel-independent quantities staged in shared memory.
template <typename T>
struct EdgeStage {
    T Y[kNumLm];              // harmonics
    T dY[3][kNumLm];          // gradients (reverse kernels only)
    T x;                      // r - h * bin
    T ux, uy, uz;             // unit vector
    long long coef_base;      // (pair * num_bins + bin) * F * 4
    long long coef_base_dir;  // the same with the ordered pair (type_i * num_elements + type_j): folded layer-0 table
    int j;                    // sender row
    int tj;                   // sender type
};

struct SplineMeta {
    double h;
    int num_bins;
    int num_elements;
};

// ---------------------------------------------------------------------------------------------
// Work distribution of the edge kernels. The grids are persistent (resident CTAs per SM x SMs) and the work items are
// handed out through a device counter, in order, so that a CTA that shares its SM with fewer others, or drew shorter
// items, simply takes more of them: with a static split the kernel lasts as long as the CTA with the most items
// (4000 receivers over 444 CTAs: ten rounds for an average of nine). sched[0] = next item, sched[1] = CTAs that have left;
// the last CTA to leave re-arms both, so no launch needs a memset.
// The reverse kernels write per-edge outputs only, so their item is (receiver, batch of <= kEdgeBatch of its edges, equal
// sizes), listed once per edge set by work_items_fill_kernel; measured on the 4000-atom float64 case: tensor-product reverse
// 2.01 -> 1.87 ms. The forward kernels accumulate over a receiver's edges (item = receiver) and keep the static split: with
// the counter they measured 2-3 % slower.
// ---------------------------------------------------------------------------------------------
// The item after the current one is requested when the current one starts, so the counter's latency hides behind the work;
// two slots alternate, and the barrier that ends an item orders the slot's write before its read.
__device__ __forceinline__ int work_first(int* __restrict__ sched, int (&s_next)[2]) {
    if (threadIdx.x == 0) s_next[0] = atomicAdd(sched, 1);
    __syncthreads();
    return s_next[0];
}
__device__ __forceinline__ void work_prefetch(int* __restrict__ sched, int (&s_next)[2], int& par) {
    par ^= 1;
    if (threadIdx.x == 0) s_next[par] = atomicAdd(sched, 1);
}
__device__ __forceinline__ int work_next(const int (&s_next)[2], int par) {
    __syncthreads();                 // everyone is done with the current item (shared memory); s_next[par] is written
    return s_next[par];
}
__device__ __forceinline__ void work_leave(int* __restrict__ sched) {
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(sched + 1, 1) == static_cast<int>(gridDim.x) - 1) { sched[0] = 0; sched[1] = 0; __threadfence(); }
    }
}
static __global__ void work_items_count_kernel(int N, const int* __restrict__ order, const long long* __restrict__ first_neigh, int* __restrict__ counts) {
    const int slot = blockIdx.x * blockDim.x + threadIdx.x;
    if (slot >= N) return;
    const int i = order ? order[slot] : slot;
    counts[slot] = static_cast<int>((first_neigh[i + 1] - first_neigh[i] + kEdgeBatch - 1) / kEdgeBatch);
}
// items[q] = (receiver, first edge relative to the receiver's row, number of edges, 0)
static __global__ void work_items_fill_kernel(int N, const int* __restrict__ order, const long long* __restrict__ first_neigh,
                                              const int* __restrict__ item_ptr, int4* __restrict__ items, int* __restrict__ n_items) {
    const int slot = blockIdx.x * blockDim.x + threadIdx.x;
    if (slot >= N) return;
    const int i = order ? order[slot] : slot;
    const int deg = static_cast<int>(first_neigh[i + 1] - first_neigh[i]);
    const int nb = (deg + kEdgeBatch - 1) / kEdgeBatch;
    const int size = nb ? (deg + nb - 1) / nb : 0;
    for (int b = 0; b < nb; ++b) {
        const int begin = b * size;
        items[item_ptr[slot] + b] = make_int4(i, begin, deg - begin < size ? deg - begin : size, 0);
    }
    if (slot == N - 1) *n_items = item_ptr[slot] + nb;
}

// Fill stage[e] for the edges [e0, e0 + nb) of node i; executed by threads 0..nb-1.
template <typename T, bool GRAD>
__device__ __forceinline__ void stage_edge(EdgeStage<T>& s, long long edge, int type_i, const int* __restrict__ neigh_indices,
                                           const int* __restrict__ neigh_types, const double* __restrict__ xyz,
                                           const double* __restrict__ r, const SplineMeta sm, int F) {
    const double rr = r[edge];
    const double inv = 1.0 / rr;
    const double ax = xyz[3 * edge] * inv, ay = xyz[3 * edge + 1] * inv, az = xyz[3 * edge + 2] * inv;
    s.ux = T(ax); s.uy = T(ay); s.uz = T(az);
    real_sh3<T, GRAD>(T(ax), T(ay), T(az), T(inv), s.Y, s.dY);
    // bin and offset exactly as CubicSplineSet::evaluate_derivs (cubic_spline_set.cpp:55-56),
    // clamped to the last interval so that r within rounding of r_cut stays inside the table
    int bin = static_cast<int>(rr / sm.h);
    bin = bin < 0 ? 0 : (bin > sm.num_bins - 1 ? sm.num_bins - 1 : bin);
    s.x = T(rr - sm.h * bin);
    const int tj = neigh_types[edge];
    s.tj = tj;
    s.j = neigh_indices[edge];
    const int lo = type_i <= tj ? type_i : tj, hi = type_i <= tj ? tj : type_i;
    const int pair = lo * (2 * sm.num_elements - lo - 1) / 2 + hi;   // mace.cpp:81-83
    s.coef_base = (static_cast<long long>(pair) * sm.num_bins + bin) * F * 4;
    s.coef_base_dir = (static_cast<long long>(type_i * sm.num_elements + tj) * sm.num_bins + bin) * F * 4;
}

// ---------------------------------------------------------------------------------------------
// Folded layer-0 table. A0[i, lm, k'] = sum_k Phi0[i, lm, k] W[a][l][k, k'] with Phi0 a sum over edges of
// R0_ab(r)[l, k] Y[lm] H0[b, k] (a, b = receiver, sender type). The spline is linear in its coefficients, so
//   c'[(a, b), bin, l, k', q] = sum_k c[pair(a, b), bin, l, k, q] H0[b, k] W[a][l][k, k']        (q = 0..3)
// is again a table of cubics, per ordered pair, whose edge sum is A0 itself (the reference's device code folds the same
// two factors into its table, mace_kokkos.cpp). Built once per model in float64 from the file's numbers and stored in the
// evaluator's precision and row layout. One CTA per (a, b, bin, l), thread = output channel k'.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void fold_layer0_kernel(int E, int bins, int K, const double* __restrict__ coef /* [pairs][bins][4][K][4] */,
                                   const double* __restrict__ H0 /* [E][K] */, const double* __restrict__ W /* [E][4][K][K] */,
                                   T* __restrict__ out) {
    extern __shared__ double fold_v[];     // [K][4]: coefficients of input channel k times H0[b, k]
    const int l = blockIdx.x & 3;
    const long long rest = blockIdx.x >> 2;
    const int bin = static_cast<int>(rest % bins);
    const int ab = static_cast<int>(rest / bins);
    const int a = ab / E, b = ab % E;
    const int lo = a <= b ? a : b, hi = a <= b ? b : a;
    const int pair = lo * (2 * E - lo - 1) / 2 + hi;
    const double* in = coef + ((static_cast<size_t>(pair) * bins + bin) * 4 + l) * 4 * K;
    for (int t = threadIdx.x; t < 4 * K; t += blockDim.x) fold_v[t] = in[t] * H0[static_cast<size_t>(b) * K + (t >> 2)];
    __syncthreads();
    const double* w = W + (static_cast<size_t>(a) * 4 + l) * K * K;
    T* row = out + ((static_cast<size_t>(ab) * bins + bin) * 4 + l) * 4 * K;
    for (int kp = threadIdx.x; kp < K; kp += blockDim.x) {
        double s0 = 0, s1 = 0, s2 = 0, s3 = 0;
        for (int k = 0; k < K; ++k) {
            const double wk = w[static_cast<size_t>(k) * K + kp];
            s0 += fold_v[4 * k] * wk; s1 += fold_v[4 * k + 1] * wk; s2 += fold_v[4 * k + 2] * wk; s3 += fold_v[4 * k + 3] * wk;
        }
        if constexpr (sizeof(T) == 4) {        // rows [K][4]
            row[4 * kp] = T(s0); row[4 * kp + 1] = T(s1); row[4 * kp + 2] = T(s2); row[4 * kp + 3] = T(s3);
        } else {                               // rows [2][K][2]
            row[2 * kp] = T(s0); row[2 * kp + 1] = T(s1); row[2 * K + 2 * kp] = T(s2); row[2 * K + 2 * kp + 1] = T(s3);
        }
    }
}

// =============================================================================================
// Layer 0, forward: Phi0[i, lm, k] = sum_j R0_ab(r_ij)[l, k] * Y_ij[lm] * H0[b, k]
// (first half of MACE::compute_A0, mace.cpp:159-178, with compute_Y / compute_R0 fused in).
// =============================================================================================
template <typename T>
struct Layer0Args {
    int N, K;
    const int* node_types; const long long* first_neigh; const int* neigh_indices; const int* neigh_types;
    const double* xyz; const double* r;
    const T* coef0; SplineMeta sm;
    const T* H0_w;          // [E][K]
    // Folded table (optional): per ORDERED element pair (receiver type a, sender type b) the radial coefficients already
    // multiplied by H0[b] and by the per-type channel mix W[a][l] (fold_layer0_kernel), so that the edge sum gives A0
    // directly: Phi0 / Phi0_adj then point at A0 / A0_adj and the two channel-mixing GEMMs of layer 0 are not run.
    const T* coef0_folded;
    // Optional processing order of the receivers (node ids sorted by element type). All CTAs then work on receivers of
    // one type at a time, whose edges touch only the pair tables of that type: for configs[1] 5 of 15 tables (73 MB of
    // 220 MB), which stay resident in the 126 MB L2 instead of being re-fetched from HBM.
    const int* order;
    T* Phi0;                // [N][16][K]          (forward output)
    const T* Phi0_adj;      // [N][16][K]          (reverse input)
    double* node_forces;    // [3 * num_edges]     (reverse: accumulated into)
    int* sched;             // work counters (see work_first)
    const int4* items;      // reverse kernel: (receiver, first edge, edges) batches
    const int* n_items;
};

template <typename T>
__global__ void __launch_bounds__(kChannelBlock) layer0_forward_kernel(const Layer0Args<T> a) {
    __shared__ EdgeStage<T> st[kEdgeBatch];
    const int F = (kLmaxSH + 1) * a.K;
    for (int slot = blockIdx.x; slot < a.N; slot += gridDim.x)
    for (int kc = 0; kc < a.K; kc += blockDim.x) {
        const int i = a.order ? a.order[slot] : slot;     // nodes in element-type order: see Layer0Args::order
        const int k = kc + threadIdx.x;
        const bool active = k < a.K;
        const long long e_begin = a.first_neigh[i], e_end = a.first_neigh[i + 1];
        const int type_i = a.node_types[i];
        T acc[kNumLm];
#pragma unroll
        for (int lm = 0; lm < kNumLm; ++lm) acc[lm] = T(0);
        for (long long e0 = e_begin; e0 < e_end; e0 += kEdgeBatch) {
            const int nb = static_cast<int>(e_end - e0 < kEdgeBatch ? e_end - e0 : kEdgeBatch);
            __syncthreads();
            if (threadIdx.x < nb)
                stage_edge<T, false>(st[threadIdx.x], e0 + threadIdx.x, type_i, a.neigh_indices, a.neigh_types, a.xyz, a.r, a.sm, F);
            __syncthreads();
            if (active) {
                for (int e = 0; e < nb; ++e) {
                    const EdgeStage<T>& s = st[e];
                    const T h0 = a.coef0_folded ? T(1) : a.H0_w[s.tj * a.K + k];
                    const T x = s.x;
                    const T* cb = a.coef0_folded ? a.coef0_folded + s.coef_base_dir : a.coef0 + s.coef_base;
#pragma unroll
                    for (int l = 0; l <= kLmaxSH; ++l) {
                        const Vec4<T> c = load_coef<T>(cb + 4 * l * a.K, k, a.K);
                        const T R = (c.x + x * (c.y + x * (c.z + x * c.w))) * h0;
#pragma unroll
                        for (int lm = l * l; lm < (l + 1) * (l + 1); ++lm) acc[lm] += R * s.Y[lm];
                    }
                }
            }
        }
        if (active) {
            T* out = a.Phi0 + (static_cast<size_t>(i) * kNumLm) * a.K + k;
#pragma unroll
            for (int lm = 0; lm < kNumLm; ++lm) out[static_cast<size_t>(lm) * a.K] = acc[lm];
        }
    }
}

// =============================================================================================
// Layer 0, reverse: per-edge partial forces
//   nf[ij] -= sum_{lm,k} Phi0_adj[i,lm,k] H0[b,k] (xhat R0'[l,k] Y[lm] + R0[l,k] grad Y[lm])
// (second half of MACE::reverse_A0, mace.cpp:238-269).
// =============================================================================================
// CPT channels per thread (k, k + blockDim.x, ...): the per-edge sums over channels (16 harmonic adjoints + 1 radial
// adjoint, reduced across the warp with shuffles and across warps through shared memory) are what this kernel spends
// most of its instructions on, and a thread that adds up CPT channels before the reduction needs 1 / CPT of them.
template <typename T, int CPT>
__global__ void __launch_bounds__(kChannelBlock) layer0_reverse_kernel(const Layer0Args<T> a) {
    __shared__ EdgeStage<T> st[kEdgeBatch];
    __shared__ T red[kMaxWarps][kEdgeBatch][17];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int F = (kLmaxSH + 1) * a.K;
    __shared__ int s_next[2];
    int par = 0;
    const int n_items = *a.n_items;
    for (int item = work_first(a.sched, s_next); item < n_items; item = work_next(s_next, par))
    for (int kc = 0; kc < a.K; kc += CPT * blockDim.x) {
        if (kc == 0) work_prefetch(a.sched, s_next, par);     // ask for the next item while this one is computed
        const int4 it = a.items[item];                    // one batch of one receiver's edges, receivers in element-type order
        const int i = it.x;
        int kk[CPT];
        bool active[CPT];
#pragma unroll
        for (int c = 0; c < CPT; ++c) { kk[c] = kc + c * blockDim.x + threadIdx.x; active[c] = kk[c] < a.K; }
        const long long e_begin = a.first_neigh[i] + it.y, e_end = e_begin + it.z;
        const int type_i = a.node_types[i];
        T d[CPT][kNumLm];
#pragma unroll
        for (int c = 0; c < CPT; ++c)
#pragma unroll
            for (int lm = 0; lm < kNumLm; ++lm)
                d[c][lm] = active[c] ? a.Phi0_adj[(static_cast<size_t>(i) * kNumLm + lm) * a.K + kk[c]] : T(0);
        for (long long e0 = e_begin; e0 < e_end; e0 += kEdgeBatch) {
            const int nb = static_cast<int>(e_end - e0 < kEdgeBatch ? e_end - e0 : kEdgeBatch);
            __syncthreads();
            if (threadIdx.x < nb)
                stage_edge<T, true>(st[threadIdx.x], e0 + threadIdx.x, type_i, a.neigh_indices, a.neigh_types, a.xyz, a.r, a.sm, F);
            __syncthreads();
            for (int e = 0; e < nb; ++e) {
                const EdgeStage<T>& s = st[e];
                T W[kNumLm], fr = 0;     // adjoints of the harmonics and of the edge length, summed over this thread's channels
#pragma unroll
                for (int lm = 0; lm < kNumLm; ++lm) W[lm] = T(0);
                const T x = s.x;
                const T* cb = a.coef0_folded ? a.coef0_folded + s.coef_base_dir : a.coef0 + s.coef_base;
#pragma unroll
                for (int c = 0; c < CPT; ++c) {
                    if (!active[c]) continue;
                    const T h0 = a.coef0_folded ? T(1) : a.H0_w[s.tj * a.K + kk[c]];
#pragma unroll
                    for (int l = 0; l <= kLmaxSH; ++l) {
                        const Vec4<T> cf = load_coef<T>(cb + 4 * l * a.K, kk[c], a.K);
                        const T R = (cf.x + x * (cf.y + x * (cf.z + x * cf.w))) * h0;
                        const T Rd = (cf.y + x * (T(2) * cf.z + T(3) * x * cf.w)) * h0;
                        T sv = 0;
#pragma unroll
                        for (int lm = l * l; lm < (l + 1) * (l + 1); ++lm) {
                            sv += d[c][lm] * s.Y[lm];
                            W[lm] += R * d[c][lm];
                        }
                        fr += Rd * sv;
                    }
                }
                int idx;
                const T wsum = warp_reduce_scatter16(W, lane, idx);
                fr = warp_sum(fr);
                if ((lane & 1) == 0) red[warp][e][idx] = wsum;
                if (lane == 0) red[warp][e][16] = fr;
            }
            __syncthreads();
            if (threadIdx.x < nb) {
                const int e = threadIdx.x;
                finish_edge_force<T, kEdgeBatch>(red, nwarps, e, st[e].dY[0], st[e].dY[1], st[e].dY[2], st[e].ux, st[e].uy, st[e].uz,
                                                 a.node_forces + 3 * (e0 + e));
            }
        }
    }
    work_leave(a.sched);
}

// =============================================================================================
// Layer 1 tensor product. Per (edge, channel):
//     Phi1[i, (l m e_p), k] += R1_p(r_ij)[k] * sum_{m1 m2} C^{l m}_{l1 m1, l2 m2} Y_ij[l1 m1] H1[j, (l2 m2), k]
// which is the reference's two-step form (Phi1r, then the Clebsch-Gordan COO contraction,
// mace.cpp:453-502) with the sums merged; Phi1r is never formed. The non-zeros of the coupling are
// written out as straight-line code (generated/tp_L*_forward.inc), so the accumulators stay in
// registers and the coupling constants are immediates; the only shared-memory traffic per edge is
// the 16 harmonics. Any per-path scale of a model file's coupling table is folded into R1_p at load.
// =============================================================================================
template <typename T>
struct TPArgs {
    int N, K;
    const int* node_types; const long long* first_neigh; const int* neigh_indices; const int* neigh_types;
    const double* xyz; const double* r;
    const T* coef1; SplineMeta sm;
    const T* H;             // sender features [rows][nLM][K]
    T* Phi1;                // forward output [N][Q][K]
    const T* dPhi1;         // reverse input  [N][Q][K]
    T* Hmsg;                // reverse output [num_edges][nLM][K]: adjoint message of each edge to its sender (float64)
    T* H_adj;               // float32: the messages are added straight into H_adj[sender] with red.global.add
    double* node_forces;    // reverse: accumulated into
    int* status;            // set non-zero by a bounded wait that ran out (staged reverse kernel)
    const int* order;       // optional processing order of the receivers (see Layer0Args::order)
    // Run-time radial mode: the radial functions of every edge (and their derivatives, reverse pass) evaluated from the
    // un-splined network by radial_hidden_kernel + a tensor-core GEMM, [num_edges][P * K]; null: cubic splines (coef1).
    const T* R_edge;
    const T* Rd_edge;
    int* sched;             // work counters (see work_first)
    const int4* items;      // reverse kernels: (receiver, first edge, edges) batches
    const int* n_items;
};

// Resident CTAs per SM the compiler is asked to allow for (register budget): measured best on B200 for the
// configs[1] model -- float64 forward 3 (168 registers), reverse 1 (no spills); float32 forward 5, reverse 4.
// For L_max = 2 the register demand is about twice as high: float32 forward 4 (128 registers, no spills; measured
// 19 % faster than 3), reverse 2; float64 1 / 1.
#ifndef SMX_L2_F32_FWD
#define SMX_L2_F32_FWD 4
#endif
#ifndef SMX_L2_F32_REV
#define SMX_L2_F32_REV 2
#endif
template <typename T> constexpr int tp_min_blocks(int LF, bool reverse) {
    if (LF >= 2) return sizeof(T) == 8 ? 1 : (reverse ? SMX_L2_F32_REV : SMX_L2_F32_FWD);
    return sizeof(T) == 8 ? (reverse ? 1 : 3) : (reverse ? 4 : 5);
}

template <typename T, int LF>
__global__ void __launch_bounds__(kChannelBlock, tp_min_blocks<T>(LF, false)) tp_forward_kernel(const TPArgs<T> a) {
    constexpr TPTable tp = make_tp_table(LF);
    __shared__ EdgeStage<T> st[kEdgeBatch];
    const int F = tp.P * a.K;
    for (int slot = blockIdx.x; slot < a.N; slot += gridDim.x)
    for (int kc = 0; kc < a.K; kc += blockDim.x) {
        const int i = a.order ? a.order[slot] : slot;     // nodes in element-type order: see Layer0Args::order
        const int k = kc + threadIdx.x;
        const bool active = k < a.K;
        const long long e_begin = a.first_neigh[i], e_end = a.first_neigh[i + 1];
        const int type_i = a.node_types[i];
        T acc[tp.Q];
#pragma unroll
        for (int q = 0; q < tp.Q; ++q) acc[q] = T(0);
        for (long long e0 = e_begin; e0 < e_end; e0 += kEdgeBatch) {
            const int nb = static_cast<int>(e_end - e0 < kEdgeBatch ? e_end - e0 : kEdgeBatch);
            __syncthreads();
            if (threadIdx.x < nb)
                stage_edge<T, false>(st[threadIdx.x], e0 + threadIdx.x, type_i, a.neigh_indices, a.neigh_types, a.xyz, a.r, a.sm, F);
            __syncthreads();
            if (active) {
                for (int e = 0; e < nb; ++e) {
                    const EdgeStage<T>& s = st[e];
                    const T x = s.x;
                    const T* cb = a.coef1 + s.coef_base;
                    const T* hrow = a.H + static_cast<size_t>(s.j) * tp.nLM * a.K + k;
                    T h[tp.nLM], R[tp.P], Y[kNumLm];
#pragma unroll
                    for (int lm2 = 0; lm2 < tp.nLM; ++lm2) h[lm2] = __ldg(hrow + static_cast<size_t>(lm2) * a.K);
                    if (a.R_edge) {
                        const T* re = a.R_edge + static_cast<size_t>(e0 + e) * F + k;
#pragma unroll
                        for (int p = 0; p < tp.P; ++p) R[p] = __ldcs(re + static_cast<size_t>(p) * a.K);
                    } else {
#pragma unroll
                        for (int p = 0; p < tp.P; ++p) {
                            const Vec4<T> c = load_coef<T>(cb + 4 * p * a.K, k, a.K);
                            R[p] = c.x + x * (c.y + x * (c.z + x * c.w));
                        }
                    }
#pragma unroll
                    for (int lm = 0; lm < kNumLm; ++lm) Y[lm] = s.Y[lm];
                    if constexpr (LF == 0) {
#include "generated/tp_L0_forward.inc"
                    } else if constexpr (LF == 1) {
#include "generated/tp_L1_forward.inc"
                    } else if constexpr (LF == 2) {
#include "generated/tp_L2_forward.inc"
                    } else {
#include "generated/tp_L3_forward.inc"
                    }
                }
            }
        }
        if (active) {
            T* out = a.Phi1 + static_cast<size_t>(i) * tp.Q * a.K + k;
#pragma unroll
            for (int q = 0; q < tp.Q; ++q) __stcs(out + static_cast<size_t>(q) * a.K, acc[q]);   // written once, read by the GEMM: stream past L2 residents
        }
    }
}

// Reverse of the tensor product (MACE::reverse_Phi1, mace.cpp:504-605) for one receiver per CTA.
// Per (edge, channel) the generated code (generated/tp_L*_reverse.inc) produces the three adjoints of
// the trilinear form: msg = dE/dH1_j (written to Hmsg, summed per sender afterwards), W = dE/dY_ij and
// fr = dE/dr_ij. W and fr are summed over channels (warp reduce-scatter, then across warps in shared
// memory) and one thread per edge turns them into the partial force
//   nf[ij] -= xhat * fr + sum_lm W[lm] * grad Y[lm].
//
// STAGED = true: the spline row of every edge (4*P*K values, 40 KB in float64 for K = 128, L_max = 1) is brought
// into shared memory by one bulk asynchronous copy (TMA) that a single thread starts one edge ahead of its use,
// through two slots guarded by a full/empty mbarrier pair each, so the coefficient reads are shared-memory loads
// instead of global loads that only 8 resident warps per SM would have to cover. A bounded wait that runs out
// sets *status, stops further copies and waits, and the kernel finishes (with results the host discards).
template <typename T, bool STAGED> constexpr int tp_reverse_batch() { return STAGED ? (sizeof(T) == 8 ? 24 : 16) : kEdgeBatch; }

template <typename T, int LF, bool STAGED>
__global__ void __launch_bounds__(kChannelBlock, tp_min_blocks<T>(LF, true)) tp_reverse_kernel(const TPArgs<T> a) {
    constexpr TPTable tp = make_tp_table(LF);
    constexpr int EB = tp_reverse_batch<T, STAGED>();
    __shared__ EdgeStage<T> st[EB];
    __shared__ T red[kMaxWarps][EB][17];
    __shared__ __align__(8) unsigned long long full_bar[2], empty_bar[2];
    __shared__ int failed;
    extern __shared__ __align__(128) unsigned char tp_dyn_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int F = tp.P * a.K;
    unsigned full_par = 0, empty_par = 0;     // bit s: parity of the phase slot s is in
    if constexpr (STAGED) {
        if (threadIdx.x == 0) {
            failed = 0;
            mbar_init(&full_bar[0], 1); mbar_init(&full_bar[1], 1);
            mbar_init(&empty_bar[0], blockDim.x); mbar_init(&empty_bar[1], blockDim.x);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncthreads();
    }
    // Work items: the row-staging variant walks whole receivers (static split; its copies run ahead inside a receiver's
    // edge list), the plain variant takes (receiver, batch) items from the work counter.
    __shared__ int s_next[2];
    int par = 0;
    const int n_work = STAGED ? a.N : *a.n_items;
    for (int w = STAGED ? static_cast<int>(blockIdx.x) : work_first(a.sched, s_next); w < n_work;
         w = STAGED ? w + static_cast<int>(gridDim.x) : work_next(s_next, par))
    for (int kc = 0; kc < a.K; kc += blockDim.x) {
        if constexpr (!STAGED) { if (kc == 0) work_prefetch(a.sched, s_next, par); }     // ask for the next item while this one is computed
        int i;
        long long e_begin, e_end;
        if constexpr (STAGED) {
            i = a.order ? a.order[w] : w;                 // nodes in element-type order: see Layer0Args::order
            e_begin = a.first_neigh[i]; e_end = a.first_neigh[i + 1];
        } else {
            const int4 it = a.items[w];
            i = it.x;
            e_begin = a.first_neigh[i] + it.y; e_end = e_begin + it.z;
        }
        const int k = kc + threadIdx.x;
        const bool active = k < a.K;
        const int Kc = a.K - kc < static_cast<int>(blockDim.x) ? a.K - kc : static_cast<int>(blockDim.x);
        T* const slot0 = reinterpret_cast<T*>(tp_dyn_smem);
        T* const slot1 = slot0 + 4 * tp.P * Kc;
        const int type_i = a.node_types[i];
        T d[tp.Q];
#pragma unroll
        for (int q = 0; q < tp.Q; ++q)
            d[q] = active ? __ldcs(a.dPhi1 + (static_cast<size_t>(i) * tp.Q + q) * a.K + k) : T(0);
        for (long long e0 = e_begin; e0 < e_end; e0 += EB) {
            const int nb = static_cast<int>(e_end - e0 < EB ? e_end - e0 : EB);
            __syncthreads();
            if (threadIdx.x < nb)
                stage_edge<T, true>(st[threadIdx.x], e0 + threadIdx.x, type_i, a.neigh_indices, a.neigh_types, a.xyz, a.r, a.sm, F);
            __syncthreads();
            if constexpr (STAGED) {
                if (threadIdx.x == 0 && !failed) {
                    issue_row_copy<T>(slot0, a.coef1 + st[0].coef_base, tp.P, a.K, kc, Kc, &full_bar[0]);
                    if (nb > 1) issue_row_copy<T>(slot1, a.coef1 + st[1].coef_base, tp.P, a.K, kc, Kc, &full_bar[1]);
                }
            }
            for (int e = 0; e < nb; ++e) {
                const EdgeStage<T>& s = st[e];
                T W[kNumLm], fr;      // assigned by the generated code (first contribution of each entry), zero for idle lanes
                const int sl = e & 1;
                T R[tp.P], Rd[tp.P];
                if constexpr (STAGED) {
                    if (!*reinterpret_cast<volatile int*>(&failed)) {
                        if (!mbar_wait(&full_bar[sl], (full_par >> sl) & 1u)) { failed = 1; atomicMax(a.status, 3); }
                    }
                    full_par ^= 1u << sl;
                    const T* slot = sl ? slot1 : slot0;
                    const T x = s.x;
                    if (active) {
#pragma unroll
                        for (int p = 0; p < tp.P; ++p) {
                            const Vec4<T> c = lds_coef<T>(slot, p, threadIdx.x, Kc);
                            R[p] = c.x + x * (c.y + x * (c.z + x * c.w));
                            Rd[p] = c.y + x * (T(2) * c.z + T(3) * x * c.w);
                        }
                    }
                    mbar_arrive(&empty_bar[sl]);                 // this thread has read its part of the slot
                    if (threadIdx.x == 0) {
                        if (e + 2 < nb && !failed) {
                            if (!mbar_wait(&empty_bar[sl], (empty_par >> sl) & 1u)) { failed = 1; atomicMax(a.status, 4); }
                            else issue_row_copy<T>(sl ? slot1 : slot0, a.coef1 + st[e + 2].coef_base, tp.P, a.K, kc, Kc, &full_bar[sl]);
                        }
                    }
                    empty_par ^= 1u << sl;
                }
                if (active) {
                    const T x = s.x;
                    const T* hrow = a.H + static_cast<size_t>(s.j) * tp.nLM * a.K + k;
                    T h[tp.nLM], msg[tp.nLM], Y[kNumLm];
#pragma unroll
                    for (int lm2 = 0; lm2 < tp.nLM; ++lm2) h[lm2] = __ldg(hrow + static_cast<size_t>(lm2) * a.K);
                    if constexpr (!STAGED) {
                        if (a.R_edge) {
                            const T* re = a.R_edge + static_cast<size_t>(e0 + e) * F + k;
                            const T* rde = a.Rd_edge + static_cast<size_t>(e0 + e) * F + k;
#pragma unroll
                            for (int p = 0; p < tp.P; ++p) { R[p] = __ldcs(re + static_cast<size_t>(p) * a.K); Rd[p] = __ldcs(rde + static_cast<size_t>(p) * a.K); }
                        } else {
                            const T* cb = a.coef1 + s.coef_base;
#pragma unroll
                            for (int p = 0; p < tp.P; ++p) {
                                const Vec4<T> c = load_coef<T>(cb + 4 * p * a.K, k, a.K);
                                R[p] = c.x + x * (c.y + x * (c.z + x * c.w));
                                Rd[p] = c.y + x * (T(2) * c.z + T(3) * x * c.w);
                            }
                        }
                    }
#pragma unroll
                    for (int lm = 0; lm < kNumLm; ++lm) Y[lm] = s.Y[lm];
                    if constexpr (LF == 0) {
#include "generated/tp_L0_reverse.inc"
                    } else if constexpr (LF == 1) {
#include "generated/tp_L1_reverse.inc"
                    } else if constexpr (LF == 2) {
#include "generated/tp_L2_reverse.inc"
                    } else {
#include "generated/tp_L3_reverse.inc"
                    }
                    if constexpr (sizeof(T) == 8) {
                        // float64: deterministic two-step scatter (per-edge message, then a fixed-order sum per sender)
                        T* mrow = a.Hmsg + static_cast<size_t>(e0 + e) * tp.nLM * a.K + k;
#pragma unroll
                        // streaming stores: the message buffer is written once and read once (sender_gather) and must not
                        // push the spline tables out of L2
                        for (int lm2 = 0; lm2 < tp.nLM; ++lm2) __stcs(mrow + static_cast<size_t>(lm2) * a.K, msg[lm2]);
                    } else {
                        // float32: one reduction per value directly into the sender's row (no message buffer)
                        T* arow = a.H_adj + static_cast<size_t>(s.j) * tp.nLM * a.K + k;
#pragma unroll
#ifdef SMX_TIMING_ONLY_NO_SCATTER      // measurement builds only: what the reductions into the senders' rows cost (results are wrong)
                        if (msg[0] == T(1.2345e30))
#endif
                        for (int lm2 = 0; lm2 < tp.nLM; ++lm2) atomicAdd(arow + static_cast<size_t>(lm2) * a.K, msg[lm2]);
                    }
                } else {
#pragma unroll
                    for (int lm = 0; lm < kNumLm; ++lm) W[lm] = T(0);
                    fr = T(0);
                }
                int idx;
                const T wsum = warp_reduce_scatter16(W, lane, idx);
                fr = warp_sum(fr);
                if ((lane & 1) == 0) red[warp][e][idx] = wsum;
                if (lane == 0) red[warp][e][16] = fr;
            }
            __syncthreads();
            if (threadIdx.x < nb) {
                const int e = threadIdx.x;
                finish_edge_force<T, EB>(red, nwarps, e, st[e].dY[0], st[e].dY[1], st[e].dY[2], st[e].ux, st[e].uy, st[e].uz,
                                         a.node_forces + 3 * (e0 + e));
            }
        }
    }
    if constexpr (!STAGED) work_leave(a.sched);
    if constexpr (STAGED) {
        // after a failed wait: give copies that may still be in flight one more bounded wait before the CTA exits
        __syncthreads();
        if (threadIdx.x == 0 && failed) {
            mbar_wait(&full_bar[0], (full_par & 1u) ^ 1u);
            mbar_wait(&full_bar[1], ((full_par >> 1) & 1u) ^ 1u);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// float64 reverse of the tensor product with the receiver's adjoint in tensor memory.
//
// tp_reverse_kernel<double> keeps d[Q] (the adjoint of the receiver's tensor product, 2 registers per value: 80 registers
// for Q = 40) in registers for the whole walk over the receiver's edges; with the 16 harmonic adjoints, the messages, the
// radial values and the coupling temporaries that is 254 registers, i.e. two resident CTAs (8 warps) per SM, too few to
// cover the latency of the coefficient loads that start every edge. Blackwell's tensor memory (TMEM, 512 columns x 128
// lanes x 32 bits per SM, normally the accumulator of tcgen05.mma) is used here as a per-thread scratchpad instead: thread
// t of the CTA owns TMEM lane t and keeps its d values there (tcgen05.st once per receiver), fetching the 2l+1 values of
// one path at a time (tcgen05.ld) while it works on the previous path. TMEM has its own data path, so this costs neither
// registers nor shared-memory / L1 bandwidth, which the coefficient stream needs. The register budget then allows three
// resident CTAs per SM.
//
// Column layout (per lane): path p starts at tp_tmem_col(p), aligned to its padded width (2, 8, 16 or 16 columns for
// l = 0, 1, 2, 3; a double takes two 32-bit columns). A CTA allocates the next power of two >= the total; the host
// checks that the resident CTAs of one SM fit into the 512 columns.
// ---------------------------------------------------------------------------------------------
constexpr int tp_tmem_width(int l) { return l == 0 ? 2 : (l == 1 ? 8 : 16); }
constexpr int tp_tmem_col(const TPTable& tp, int p) {
    int col = 0;
    for (int q = 0; q < p; ++q) {
        const int w = tp_tmem_width(tp.l[q]);
        col = (col + w - 1) / w * w + w;
    }
    const int w = tp_tmem_width(tp.l[p]);
    return (col + w - 1) / w * w;
}
constexpr int tp_tmem_cols(int LF) {
    const TPTable tp = make_tp_table(LF);
    const int used = tp_tmem_col(tp, tp.P - 1) + tp_tmem_width(tp.l[tp.P - 1]);
    int alloc = 32;
    while (alloc < used) alloc *= 2;
    return alloc;
}

// Starts the asynchronous fetch of W 32-bit columns of this thread's TMEM lane into `v` (W = 2, 8 or 16).
template <int W>
__device__ __forceinline__ void tmem_ld_issue(uint32_t taddr, uint32_t (&v)[16]) {
    if constexpr (W == 2) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];" : "=r"(v[0]), "=r"(v[1]) : "r"(taddr) : "memory");
    } else if constexpr (W == 8) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                     : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]) : "r"(taddr) : "memory");
    } else {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                     : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                       "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]) : "r"(taddr) : "memory");
    }
}
// Waits for the fetches this thread started; the registers are operands so that no use of them moves above the wait.
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&v)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]), "+r"(v[9]),
                   "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]) :: "memory");
}
__device__ __forceinline__ void tmem_st2(uint32_t taddr, double x) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x2.b32 [%0], {%1, %2};" ::"r"(taddr), "r"(__double2loint(x)), "r"(__double2hiint(x)) : "memory");
}

template <int LF, int MINB>
__global__ void __launch_bounds__(kChannelBlock, MINB) tp_reverse_tmem_kernel(const TPArgs<double> a) {
    using T = double;
    constexpr TPTable tp = make_tp_table(LF);
    constexpr int EB = kEdgeBatch;
    constexpr int kCols = tp_tmem_cols(LF);
    __shared__ EdgeStage<T> st[EB];
    __shared__ T red[kMaxWarps][EB][17];
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int F = tp.P * a.K;
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(kCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // this thread's lane: 32 * (warp % 4) + lane, in bits 16.. of the address (a warp reaches the 32 lanes of its quadrant)
    const uint32_t tbase = tmem_slot + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    // two sets of staging registers, used by the paths of even and odd index: the set a path has just consumed is dead
    // until the path after the next one refills it, so its registers can become the path's double-precision values in place
    uint32_t stage0[16], stage1[16];
#pragma unroll
    for (int q = 0; q < 16; ++q) { stage0[q] = 0u; stage1[q] = 0u; }

    __shared__ int s_next[2];
    int par = 0;
    const int n_items = *a.n_items;
    for (int item = work_first(a.sched, s_next); item < n_items; item = work_next(s_next, par))
    for (int kc = 0; kc < a.K; kc += blockDim.x) {
        if (kc == 0) work_prefetch(a.sched, s_next, par);     // ask for the next item while this one is computed
        const int4 it = a.items[item];                    // one batch of one receiver's edges, receivers in element-type order
        const int i = it.x;
        const bool active = kc + static_cast<int>(threadIdx.x) < a.K;
        const int k = active ? kc + threadIdx.x : a.K - 1;     // idle lanes shadow the last channel with a zero adjoint: the
                                                               // tensor-memory instructions need the whole warp
        const long long e_begin = a.first_neigh[i] + it.y, e_end = e_begin + it.z;
        const int type_i = a.node_types[i];
        // the receiver's adjoint into this thread's TMEM lane, path by path
        static_for<tp.P>([&](auto pc) {
            constexpr int p = decltype(pc)::value;
            constexpr int col = tp_tmem_col(tp, p);
#pragma unroll
            for (int m = 0; m < 2 * tp.l[p] + 1; ++m) {
                const T v = active ? __ldcs(a.dPhi1 + (static_cast<size_t>(i) * tp.Q + tp.lme(p, m)) * a.K + k) : T(0);
                tmem_st2(tbase + col + 2 * m, v);
            }
        });
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tmem_ld_issue<tp_tmem_width(tp.l[0])>(tbase + tp_tmem_col(tp, 0), stage0);     // path 0 of the first edge
        for (long long e0 = e_begin; e0 < e_end; e0 += EB) {
            const int nb = static_cast<int>(e_end - e0 < EB ? e_end - e0 : EB);
            __syncthreads();
            if (threadIdx.x < nb)
                stage_edge<T, true>(st[threadIdx.x], e0 + threadIdx.x, type_i, a.neigh_indices, a.neigh_types, a.xyz, a.r, a.sm, F);
            __syncthreads();
            for (int e = 0; e < nb; ++e) {
                const EdgeStage<T>& s = st[e];
                T W[kNumLm], fr;      // assigned by the generated code (first contribution of each entry)
                T R[tp.P], Rd[tp.P];
                const T x = s.x;
                const T* hrow = a.H + static_cast<size_t>(s.j) * tp.nLM * a.K + k;
                T h[tp.nLM], msg[tp.nLM], Y[kNumLm];
#pragma unroll
                for (int lm2 = 0; lm2 < tp.nLM; ++lm2) h[lm2] = __ldg(hrow + static_cast<size_t>(lm2) * a.K);
                const T* cb = a.coef1 + s.coef_base;
#pragma unroll
                for (int p = 0; p < tp.P; ++p) {
                    const Vec4<T> c = load_coef<T>(cb + 4 * p * a.K, k, a.K);
                    R[p] = c.x + x * (c.y + x * (c.z + x * c.w));
                    Rd[p] = c.y + x * (T(2) * c.z + T(3) * x * c.w);
                }
#pragma unroll
                for (int lm = 0; lm < kNumLm; ++lm) Y[lm] = s.Y[lm];
                // Path p's adjoint values arrive in `stage` (fetch started while path p - 1 was computed); they are moved
                // into dp and the fetch of the next path (path 0 again after the last: the adjoint belongs to the receiver,
                // not to the edge) starts before path p is computed.
#define TP_PATH_D(p, n, dp)                                                                                   \
                {                                                                                             \
                    uint32_t (&cur_)[16] = ((p) & 1) ? stage1 : stage0;                                       \
                    uint32_t (&nxt_)[16] = ((((p) + 1) % tp.P) & 1) ? stage1 : stage0;                        \
                    tmem_ld_wait(cur_);                                                                       \
                    _Pragma("unroll") for (int m_ = 0; m_ < (n); ++m_) dp[m_] = __hiloint2double(static_cast<int>(cur_[2 * m_ + 1]), static_cast<int>(cur_[2 * m_])); \
                    tmem_ld_issue<tp_tmem_width(tp.l[((p) + 1) % tp.P])>(tbase + tp_tmem_col(tp, ((p) + 1) % tp.P), nxt_); \
                }
                if constexpr (LF == 0) {
#include "generated/tp_L0_reverse_bypath.inc"
                } else if constexpr (LF == 1) {
#include "generated/tp_L1_reverse_bypath.inc"
                } else if constexpr (LF == 2) {
#include "generated/tp_L2_reverse_bypath.inc"
                } else {
#include "generated/tp_L3_reverse_bypath.inc"
                }
#undef TP_PATH_D
                if (active) {
                    // deterministic two-step scatter: per-edge message, then a fixed-order sum per sender (sender_gather_kernel)
                    T* mrow = a.Hmsg + static_cast<size_t>(e0 + e) * tp.nLM * a.K + k;
#pragma unroll
                    for (int lm2 = 0; lm2 < tp.nLM; ++lm2) __stcs(mrow + static_cast<size_t>(lm2) * a.K, msg[lm2]);
                }
                int idx;
                const T wsum = warp_reduce_scatter16(W, lane, idx);
                fr = warp_sum(fr);
                if ((lane & 1) == 0) red[warp][e][idx] = wsum;
                if (lane == 0) red[warp][e][16] = fr;
            }
            __syncthreads();
            if (threadIdx.x < nb) {
                const int e = threadIdx.x;
                finish_edge_force<T, EB>(red, nwarps, e, st[e].dY[0], st[e].dY[1], st[e].dY[2], st[e].ux, st[e].uy, st[e].uz,
                                         a.node_forces + 3 * (e0 + e));
            }
        }
        tmem_ld_wait(stage0);     // the fetch started after the last path of the last edge: nothing may be in flight when d is rewritten
    }
    work_leave(a.sched);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_slot), "r"(kCols) : "memory");
}

// ---------------------------------------------------------------------------------------------
// Run-time radial mode, first part: the hidden activations of the radial network and their derivatives with respect
// to the edge length, per edge. The network is what the reference's exporter tabulates into its cubic splines
// (symmetrix/source/symmetrix/extract_mace_data.py:144-172):
//   f_n(r) = sqrt(2 / r_cut) sin(n pi r / r_cut) / r * cutoff_p(r / r_cut) * pair_scale[pair][n]
//   x <- s silu(x W) per hidden layer (s = silu_scale),  dx/dr by the chain rule alongside.
// The last layer (hidden -> P K values per edge) is a dense GEMM over all edges and runs on the tensor cores
// (gemm_rows_tcgen05_kernel). One group of `hidden` threads per edge, four groups per CTA; the weights sit in shared
// memory, thread j of a group owns neuron j.
// ---------------------------------------------------------------------------------------------
struct RadialNetArgs {
    int N, num_bessel, poly_p, hidden, num_hidden_layers, num_elements;
    float r_cut, silu_scale;
    const int* node_types; const long long* first_neigh; const int* neigh_types; const double* r;
    const float* w_first;      // [num_bessel][hidden]
    const float* w_hidden;     // [num_hidden_layers - 1][hidden][hidden]
    const float* pair_scale;   // [pairs][num_bessel]
    float* x_out;              // [num_edges][hidden]
    float* dx_out;             // [num_edges][hidden]
};
constexpr int kRadialGroups = 4;

static __global__ void __launch_bounds__(kRadialGroups * 64) radial_hidden_kernel(const RadialNetArgs a) {
    extern __shared__ float radial_smem[];
    const int H = a.hidden;
    float* w1 = radial_smem;                                        // [num_bessel][H]
    float* wh = w1 + a.num_bessel * H;                              // [(layers - 1)][H][H]
    float* act = wh + (a.num_hidden_layers - 1) * H * H;            // [groups][2 buffers][2 (x, dx)][64]
    for (int t = threadIdx.x; t < a.num_bessel * H; t += blockDim.x) w1[t] = a.w_first[t];
    for (int t = threadIdx.x; t < (a.num_hidden_layers - 1) * H * H; t += blockDim.x) wh[t] = a.w_hidden[t];
    __syncthreads();
    const int group = threadIdx.x / 64, j = threadIdx.x % 64;
    float* mine = act + group * 4 * 64;
    const double pi = 3.14159265358979323846;
    for (int i = blockIdx.x; i < a.N; i += gridDim.x) {
        const int type_i = a.node_types[i];
        const long long e_begin = a.first_neigh[i], e_end = a.first_neigh[i + 1];
        const long long rounds = (e_end - e_begin + kRadialGroups - 1) / kRadialGroups;
        for (long long rd = 0; rd < rounds; ++rd) {
            const long long e = e_begin + rd * kRadialGroups + group;
            const bool live = e < e_end;
            if (live && j < a.num_bessel) {
                const double rr = a.r[e], rc = a.r_cut;
                const int tj = a.neigh_types[e];
                const int lo = type_i <= tj ? type_i : tj, hi = type_i <= tj ? tj : type_i;
                const int pair = lo * (2 * a.num_elements - lo - 1) / 2 + hi;
                const double kn = (j + 1) * pi / rc, amp = sqrt(2.0 / rc);
                double sn, cs;
                sincos(kn * rr, &sn, &cs);
                const double b = amp * sn / rr, db = amp * (kn * cs / rr - sn / (rr * rr));
                const double x = rr / rc, p = a.poly_p;
                double c = 0.0, dc = 0.0;
                if (x < 1.0) {
                    double xp1 = 1.0;                              // x^(p - 1) by repeated multiplication (p is a small integer)
                    for (int q = 1; q < a.poly_p; ++q) xp1 *= x;
                    const double xp = xp1 * x, xq = xp * x, xr = xq * x;
                    c = 1.0 - (p + 1.0) * (p + 2.0) / 2.0 * xp + p * (p + 2.0) * xq - p * (p + 1.0) / 2.0 * xr;
                    dc = (-(p + 1.0) * (p + 2.0) / 2.0 * p * xp1 + p * (p + 2.0) * (p + 1.0) * xp - p * (p + 1.0) / 2.0 * (p + 2.0) * xq) / rc;
                }
                const double sc = a.pair_scale[pair * a.num_bessel + j];
                mine[j] = static_cast<float>(b * c * sc);
                mine[64 + j] = static_cast<float>((db * c + b * dc) * sc);
            }
            __syncthreads();
            int cur = 0;
            for (int layer = 0; layer < a.num_hidden_layers; ++layer) {
                const float* xin = mine + cur * 128;
                float* xout = mine + (cur ^ 1) * 128;
                const int n_in = layer == 0 ? a.num_bessel : H;
                const float* w = layer == 0 ? w1 : wh + (layer - 1) * H * H;
                if (live && j < H) {
                    float z = 0.f, dz = 0.f;
                    for (int q = 0; q < n_in; ++q) {
                        const float wv = w[q * H + j];
                        z = fmaf(xin[q], wv, z);
                        dz = fmaf(xin[64 + q], wv, dz);
                    }
                    const float sig = 1.f / (1.f + expf(-z));
                    xout[j] = a.silu_scale * z * sig;
                    xout[64 + j] = a.silu_scale * sig * (1.f + z * (1.f - sig)) * dz;
                }
                __syncthreads();
                cur ^= 1;
            }
            if (live && j < H) {
                a.x_out[static_cast<size_t>(e) * H + j] = mine[cur * 128 + j];
                a.dx_out[static_cast<size_t>(e) * H + j] = mine[cur * 128 + 64 + j];
            }
            __syncthreads();
        }
    }
}

// Input check for callers that cannot vouch for their edge arrays: counts, per kind, the entries that would make the
// evaluation read out of bounds or produce non-finite values. Reads only inside the given arrays.
//   0 node type outside [0, num_elements)      1 negative neighbour count      2 counts do not add up to the edge total
//   3 sender index outside [0, feature_rows)   4 sender type outside the model  5 r not finite, <= 0 or beyond r_cut
//   6 r differs from |xyz| by more than 1e-6 relative
constexpr int kNumInputChecks = 7;
static __global__ void validate_inputs_kernel(int N, long long E, int num_elements, int feature_rows, double r_cut,
                                       const int* __restrict__ node_types, const int* __restrict__ num_neigh,
                                       const long long* __restrict__ first_neigh, const int* __restrict__ neigh_indices,
                                       const int* __restrict__ neigh_types, const double* __restrict__ xyz, const double* __restrict__ r,
                                       unsigned long long* __restrict__ counts) {
    const long long t0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    unsigned long long bad[kNumInputChecks] = {};
    for (long long i = t0; i < N; i += stride) {
        if (node_types[i] < 0 || node_types[i] >= num_elements) bad[0] += 1;
        if (num_neigh[i] < 0) bad[1] += 1;
    }
    if (t0 == 0 && N > 0 && first_neigh[N - 1] + num_neigh[N - 1] != E) bad[2] += 1;
    for (long long e = t0; e < E; e += stride) {
        if (neigh_indices[e] < 0 || neigh_indices[e] >= feature_rows) bad[3] += 1;
        if (neigh_types[e] < 0 || neigh_types[e] >= num_elements) bad[4] += 1;
        const double rr = r[e];
        if (!(rr > 0.0) || !(rr <= r_cut * (1.0 + 1e-12)) || !isfinite(rr)) bad[5] += 1;
        const double x = xyz[3 * e], y = xyz[3 * e + 1], z = xyz[3 * e + 2];
        const double d = sqrt(x * x + y * y + z * z);
        if (!(fabs(d - rr) <= 1e-6 * fmax(d, rr))) bad[6] += 1;
    }
    for (int c = 0; c < kNumInputChecks; ++c)
        if (bad[c]) atomicAdd(counts + c, bad[c]);
}

// Measurement probe: streams, for every edge of the current edge set, the spline row the edge kernels read
// (same (pair, bin) addressing, same per-thread 16-byte loads) and does nothing else; its duration is the
// floor the L2 -> SM path sets for one pass of an edge kernel over the edge set. No barriers and few
// registers, so the SMs run it at full occupancy.
template <typename T>
__global__ void row_stream_probe_kernel(int N, int K, int P, const int* __restrict__ node_types, const long long* __restrict__ first_neigh,
                                        const int* __restrict__ neigh_types, const double* __restrict__ r, const T* __restrict__ coef,
                                        SplineMeta sm, const int* __restrict__ order, T* __restrict__ sink) {
    T acc = T(0);
    for (int slot = blockIdx.x; slot < N; slot += gridDim.x) {
        const int i = order ? order[slot] : slot;
        const int type_i = node_types[i];
        const long long e_begin = first_neigh[i], e_end = first_neigh[i + 1];
        for (int k = threadIdx.x; k < K; k += blockDim.x)
            for (long long e = e_begin; e < e_end; ++e) {
                int bin = static_cast<int>(r[e] / sm.h);
                bin = bin < 0 ? 0 : (bin > sm.num_bins - 1 ? sm.num_bins - 1 : bin);
                const int tj = neigh_types[e];
                const int lo = type_i <= tj ? type_i : tj, hi = type_i <= tj ? tj : type_i;
                const int pair = lo * (2 * sm.num_elements - lo - 1) / 2 + hi;
                const T* row = coef + (static_cast<long long>(pair) * sm.num_bins + bin) * P * K * 4;
                for (int p = 0; p < P; ++p) {
                    const Vec4<T> c = load_coef<T>(row + 4 * p * K, k, K);
                    acc += (c.x + c.y) + (c.z + c.w);
                }
            }
    }
    if (acc == T(1.2345e30)) *sink = acc;     // never true for real tables; keeps the loads alive
}

// Sum of the adjoint messages of all edges that have row j as their sender, in the fixed order
// of the sender-sorted edge list (deterministic; takes the place of the atomic scatter the
// reference's device code uses, mace_kokkos.cpp:1008-1010):
//   H_adj[j, :, :] += sum_{e in in_edges(j)} Hmsg[e, :, :]
// VEC: a thread sums two neighbouring values with 16-byte loads (float64 rows of even width; the rows start 16-byte aligned).
template <typename T, bool VEC>
__global__ void sender_gather_kernel(int rows, int width, const long long* __restrict__ in_ptr,
                                     const int* __restrict__ in_edge, const T* __restrict__ Hmsg, T* __restrict__ H_adj) {
    for (int j = blockIdx.x; j < rows; j += gridDim.x) {
        const long long b = in_ptr[j], e = in_ptr[j + 1];
        if constexpr (VEC && sizeof(T) == 8) {
            for (int c = 2 * threadIdx.x; c < width; c += 2 * blockDim.x) {
                // eight rows in flight per thread; the additions stay in list order
                double a0 = 0, a1 = 0;
                long long n = b;
                for (; n + 8 <= e; n += 8) {
                    double2 v[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        v[u] = __ldcs(reinterpret_cast<const double2*>(Hmsg + static_cast<size_t>(in_edge[n + u]) * width + c));
#pragma unroll
                    for (int u = 0; u < 8; ++u) { a0 += v[u].x; a1 += v[u].y; }
                }
                for (; n < e; ++n) {
                    const double2 v = __ldcs(reinterpret_cast<const double2*>(Hmsg + static_cast<size_t>(in_edge[n]) * width + c));
                    a0 += v.x; a1 += v.y;
                }
                double2* out = reinterpret_cast<double2*>(H_adj + static_cast<size_t>(j) * width + c);
                double2 o = *out;
                o.x += a0; o.y += a1;
                *out = o;
            }
            continue;
        }
        for (int c = threadIdx.x; c < width; c += blockDim.x) {
            // eight rows in flight per thread; the additions stay in list order
            T acc = 0;
            long long n = b;
            for (; n + 8 <= e; n += 8) {
                T v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u] = __ldcs(Hmsg + static_cast<size_t>(in_edge[n + u]) * width + c);
#pragma unroll
                for (int u = 0; u < 8; ++u) acc += v[u];
            }
            for (; n < e; ++n) acc += __ldcs(Hmsg + static_cast<size_t>(in_edge[n]) * width + c);
            H_adj[static_cast<size_t>(j) * width + c] += acc;
        }
    }
}

// =============================================================================================
// Symmetric contraction (MACE::compute_M0 / compute_M1, mace.cpp:348-370,759-777, and their
// reverses :372-395,779-794). One thread per (node, channel) walks the nested Horner program of
// each output component; the 16 inputs of the thread live in shared memory.
// =============================================================================================
template <typename T>
struct PolyArgs {
    int N, K;
    int num_out;                 // output components (nLM for M0, 1 for M1)
    int num_mono;                // monomial rows per element in `coef`
    const int* node_types;
    const int* perm;             // nodes sorted by element type
    const int* type_seg;         // [E + 1] segment of each type in perm
    int num_types;               // E
    const int* prog;             // concatenated operation streams (see compile_polynomial)
    const int* prog_off;         // [num_out] first word of each stream
    const int* prog_cnt;         // [num_out] operations to execute (a multiple of the prefetch distance)
    const int* mono_off;         // [num_out] first coefficient row of each stream
    const T* coef;               // [E][num_mono][K]
    const T* A;                  // [N][16][K]
    T* M;                        // forward output [N][num_out][K]
    const T* M_adj;              // reverse input  [N][num_out][K]
    T* A_adj;                    // reverse output [N][16][K] (overwritten)
};

constexpr int kPolyAhead = 8;    // must equal kPolyPrefetch of the program builder

__device__ __forceinline__ int poly_kind(int w) { return w & 7; }
__device__ __forceinline__ int poly_var(int w) { return (w >> 3) & 31; }
template <typename T>
__device__ __forceinline__ T poly_coef(const T* c, int w, int K) {
    const int row = (w >> 8) - 1;
    return row >= 0 ? __ldg(c + static_cast<size_t>(row) * K) : T(0);
}

// One thread owns one channel of NB nodes of the same element type (blockIdx.y = type, blockIdx.x =
// group of NB nodes in the type's segment of the sorted node list, blockIdx.z = channel chunk), so
// every coefficient fetched from L2 is used NB times, and the operation words and coefficients of
// the next kPolyAhead operations are already in flight while one executes. Inputs live in shared
// memory as [node slot][variable][thread].
template <typename T, int NB>
__global__ void poly_forward_kernel(const PolyArgs<T> a) {
    extern __shared__ unsigned char smem_raw[];
    T* As = reinterpret_cast<T*>(smem_raw);           // [NB][16][blockDim.x]
    const int nt = blockDim.x, t = threadIdx.x;
    const int type = blockIdx.y;
    const int seg_begin = a.type_seg[type], seg_count = a.type_seg[type + 1] - seg_begin;
    const int first = blockIdx.x * NB;
    if (first >= seg_count) return;
    const int k = blockIdx.z * nt + t;
    if (k >= a.K) return;
    int node[NB];
#pragma unroll
    for (int n = 0; n < NB; ++n) {
        const bool valid = first + n < seg_count;
        node[n] = valid ? a.perm[seg_begin + first + n] : -1;
#pragma unroll
        for (int q = 0; q < kNumLm; ++q)
            As[(n * kNumLm + q) * nt + t] = valid ? a.A[(static_cast<size_t>(node[n]) * kNumLm + q) * a.K + k] : T(0);
    }
    const T* cf = a.coef + static_cast<size_t>(type) * a.num_mono * a.K + k;
    for (int o = 0; o < a.num_out; ++o) {
        const int* w = a.prog + a.prog_off[o];
        const int count = a.prog_cnt[o];
        const T* c = cf + static_cast<size_t>(a.mono_off[o]) * a.K;
        int wr[kPolyAhead];
        T cr[kPolyAhead];
#pragma unroll
        for (int u = 0; u < kPolyAhead; ++u) { wr[u] = __ldg(w + u); cr[u] = poly_coef(c, wr[u], a.K); }
        T total_v[NB], s1[NB], s2[NB];
#pragma unroll
        for (int n = 0; n < NB; ++n) total_v[n] = s1[n] = s2[n] = T(0);
        for (int base = 0; base < count; base += kPolyAhead) {
#pragma unroll
            for (int u = 0; u < kPolyAhead; ++u) {
                const int word = wr[u];
                const T cv = cr[u];
                wr[u] = __ldg(w + base + kPolyAhead + u);          // streams are padded, so this stays in bounds
                cr[u] = poly_coef(c, wr[u], a.K);
                const int kind = poly_kind(word), q = poly_var(word);
                if (kind == 0) {
#pragma unroll
                    for (int n = 0; n < NB; ++n) s2[n] += cv * As[(n * kNumLm + q) * nt + t];
                } else if (kind == 1) {
#pragma unroll
                    for (int n = 0; n < NB; ++n) s2[n] = cv;
                } else if (kind == 2) {
#pragma unroll
                    for (int n = 0; n < NB; ++n) s1[n] += s2[n] * As[(n * kNumLm + q) * nt + t];
                } else if (kind == 3) {
#pragma unroll
                    for (int n = 0; n < NB; ++n) s1[n] = cv;
                } else if (kind == 4) {
#pragma unroll
                    for (int n = 0; n < NB; ++n) total_v[n] += s1[n] * As[(n * kNumLm + q) * nt + t];
                }
            }
        }
#pragma unroll
        for (int n = 0; n < NB; ++n)
            if (node[n] >= 0) a.M[(static_cast<size_t>(node[n]) * a.num_out + o) * a.K + k] = total_v[n];
    }
}

template <typename T, int NB>
__global__ void poly_reverse_kernel(const PolyArgs<T> a) {
    extern __shared__ unsigned char smem_raw[];
    const int nt = blockDim.x, t = threadIdx.x;
    T* As = reinterpret_cast<T*>(smem_raw);           // [NB][16][nt]
    T* Gs = As + NB * kNumLm * nt;                    // [NB][16][nt] gradient accumulators
    const int type = blockIdx.y;
    const int seg_begin = a.type_seg[type], seg_count = a.type_seg[type + 1] - seg_begin;
    const int first = blockIdx.x * NB;
    if (first >= seg_count) return;
    const int k = blockIdx.z * nt + t;
    if (k >= a.K) return;
    int node[NB];
#pragma unroll
    for (int n = 0; n < NB; ++n) {
        const bool valid = first + n < seg_count;
        node[n] = valid ? a.perm[seg_begin + first + n] : -1;
#pragma unroll
        for (int q = 0; q < kNumLm; ++q) {
            As[(n * kNumLm + q) * nt + t] = valid ? a.A[(static_cast<size_t>(node[n]) * kNumLm + q) * a.K + k] : T(0);
            Gs[(n * kNumLm + q) * nt + t] = T(0);
        }
    }
    const T* cf = a.coef + static_cast<size_t>(type) * a.num_mono * a.K + k;
    for (int o = 0; o < a.num_out; ++o) {
        T seed[NB];
#pragma unroll
        for (int n = 0; n < NB; ++n) seed[n] = node[n] >= 0 ? a.M_adj[(static_cast<size_t>(node[n]) * a.num_out + o) * a.K + k] : T(0);
        const int* w = a.prog + a.prog_off[o];
        const int count = a.prog_cnt[o];
        const T* c = cf + static_cast<size_t>(a.mono_off[o]) * a.K;
        int wr[kPolyAhead];
        T cr[kPolyAhead];
#pragma unroll
        for (int u = 0; u < kPolyAhead; ++u) { wr[u] = __ldg(w + u); cr[u] = poly_coef(c, wr[u], a.K); }
        // s1/s2: values of the open head / pair brackets; a2: A[q2]; adj1/adj2: adjoints of the brackets
        T s1[NB], s2[NB], a2[NB], adj1[NB], adj2[NB];
#pragma unroll
        for (int n = 0; n < NB; ++n) s1[n] = s2[n] = a2[n] = adj1[n] = adj2[n] = T(0);
        for (int base = 0; base < count; base += kPolyAhead) {
#pragma unroll
            for (int u = 0; u < kPolyAhead; ++u) {
                const int word = wr[u];
                const T cv = cr[u];
                wr[u] = __ldg(w + base + kPolyAhead + u);
                cr[u] = poly_coef(c, wr[u], a.K);
                const int kind = poly_kind(word), q = poly_var(word);
                if (kind == 0) {
#pragma unroll
                    for (int n = 0; n < NB; ++n) {
                        s2[n] += cv * As[(n * kNumLm + q) * nt + t];
                        Gs[(n * kNumLm + q) * nt + t] += adj2[n] * cv;
                    }
                } else if (kind == 1) {
#pragma unroll
                    for (int n = 0; n < NB; ++n) { a2[n] = As[(n * kNumLm + q) * nt + t]; s2[n] = cv; adj2[n] = adj1[n] * a2[n]; }
                } else if (kind == 2) {
#pragma unroll
                    for (int n = 0; n < NB; ++n) { Gs[(n * kNumLm + q) * nt + t] += adj1[n] * s2[n]; s1[n] += s2[n] * a2[n]; }
                } else if (kind == 3) {
#pragma unroll
                    for (int n = 0; n < NB; ++n) { s1[n] = cv; adj1[n] = seed[n] * As[(n * kNumLm + q) * nt + t]; }
                } else if (kind == 4) {
#pragma unroll
                    for (int n = 0; n < NB; ++n) Gs[(n * kNumLm + q) * nt + t] += seed[n] * s1[n];
                }
            }
        }
    }
#pragma unroll
    for (int n = 0; n < NB; ++n)
        if (node[n] >= 0)
#pragma unroll
            for (int q = 0; q < kNumLm; ++q) a.A_adj[(static_cast<size_t>(node[n]) * kNumLm + q) * a.K + k] = Gs[(n * kNumLm + q) * nt + t];
}

// Straight-line variant for models whose monomial lists are the symmetry-complete ones of
// generated/poly_canon.hpp (l_max = 3, correlation 3): one thread per (node, channel), the 16 inputs and the
// 16 gradient accumulators in registers, every coefficient one load at a compile-time offset. `coef` is then
// ordered canonically, [element][canonical monomial][K]. NOUT = number of output components (1, 4 or 9).
// NB nodes of one element type share a thread: every coefficient load then feeds NB multiply-adds (the coefficient stream
// from L2, one load per multiply-add for NB = 1, is what these kernels wait for). The generated code is written for a
// type T with fma and *; here T is a short vector over the NB nodes. Grid: one thread per (node group, channel).
template <typename S, int NB>
struct PolyVec {
    S v[NB];
    __device__ __forceinline__ PolyVec() {}
    __device__ __forceinline__ PolyVec(S x) {
#pragma unroll
        for (int n = 0; n < NB; ++n) v[n] = x;
    }
};
template <typename S, int NB>
__device__ __forceinline__ PolyVec<S, NB> fma(const PolyVec<S, NB>& x, const PolyVec<S, NB>& y, const PolyVec<S, NB>& z) {
    PolyVec<S, NB> r;
#pragma unroll
    for (int n = 0; n < NB; ++n) r.v[n] = ::fma(x.v[n], y.v[n], z.v[n]);
    return r;
}
template <typename S, int NB>
__device__ __forceinline__ PolyVec<S, NB> operator*(const PolyVec<S, NB>& x, const PolyVec<S, NB>& y) {
    PolyVec<S, NB> r;
#pragma unroll
    for (int n = 0; n < NB; ++n) r.v[n] = x.v[n] * y.v[n];
    return r;
}

template <typename S, int NOUT, int NB>
__global__ void __launch_bounds__(128) poly_fixed_forward_kernel(const PolyArgs<S> a) {
    using T = PolyVec<S, NB>;
    // flat index -> (element type, group of NB nodes of that type, channel); groups of all types are numbered consecutively
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    int g = static_cast<int>(idx / a.K);
    const int k = static_cast<int>(idx - static_cast<long long>(g) * a.K);
    int type = 0, seg_begin = 0, count = 0;
    for (; type < a.num_types; ++type) {
        seg_begin = a.type_seg[type];
        count = a.type_seg[type + 1] - seg_begin;
        const int groups = (count + NB - 1) / NB;
        if (g < groups) break;
        g -= groups;
    }
    if (type == a.num_types) return;
    int node[NB];
    bool live[NB];
#pragma unroll
    for (int n = 0; n < NB; ++n) {
        const int jn = g * NB + n;
        live[n] = jn < count;
        node[n] = a.perm[seg_begin + (live[n] ? jn : count - 1)];   // an empty slot repeats the last node; its results are dropped
    }
    const S* cf = a.coef + static_cast<size_t>(type) * a.num_mono * a.K + k;
    T A[kNumLm];
#pragma unroll
    for (int q = 0; q < kNumLm; ++q)
#pragma unroll
        for (int n = 0; n < NB; ++n) A[q].v[n] = a.A[(static_cast<size_t>(node[n]) * kNumLm + q) * a.K + k];
    {
        {
            constexpr int kOff = kCanonPolyOffset[0];
            auto C = [&](int slot) { return T(__ldg(cf + static_cast<size_t>(kOff + slot) * a.K)); };
#include "generated/poly_lm0_forward.inc"
#pragma unroll
            for (int n = 0; n < NB; ++n)
                if (live[n]) a.M[(static_cast<size_t>(node[n]) * NOUT + 0) * a.K + k] = total.v[n];
        }
    }
    if constexpr (NOUT > 1) {
        {
            constexpr int kOff = kCanonPolyOffset[1];
            auto C = [&](int slot) { return T(__ldg(cf + static_cast<size_t>(kOff + slot) * a.K)); };
#include "generated/poly_lm1_forward.inc"
#pragma unroll
            for (int n = 0; n < NB; ++n)
                if (live[n]) a.M[(static_cast<size_t>(node[n]) * NOUT + 1) * a.K + k] = total.v[n];
        }
        {
            constexpr int kOff = kCanonPolyOffset[2];
            auto C = [&](int slot) { return T(__ldg(cf + static_cast<size_t>(kOff + slot) * a.K)); };
#include "generated/poly_lm2_forward.inc"
#pragma unroll
            for (int n = 0; n < NB; ++n)
                if (live[n]) a.M[(static_cast<size_t>(node[n]) * NOUT + 2) * a.K + k] = total.v[n];
        }
        {
            constexpr int kOff = kCanonPolyOffset[3];
            auto C = [&](int slot) { return T(__ldg(cf + static_cast<size_t>(kOff + slot) * a.K)); };
#include "generated/poly_lm3_forward.inc"
#pragma unroll
            for (int n = 0; n < NB; ++n)
                if (live[n]) a.M[(static_cast<size_t>(node[n]) * NOUT + 3) * a.K + k] = total.v[n];
        }
    }
    if constexpr (NOUT > 4) {
        {
            constexpr int kOff = kCanonPolyOffset[4];
            auto C = [&](int slot) { return T(__ldg(cf + static_cast<size_t>(kOff + slot) * a.K)); };
#include "generated/poly_lm4_forward.inc"
#pragma unroll
            for (int n = 0; n < NB; ++n)
                if (live[n]) a.M[(static_cast<size_t>(node[n]) * NOUT + 4) * a.K + k] = total.v[n];
        }
        {
            constexpr int kOff = kCanonPolyOffset[5];
            auto C = [&](int slot) { return T(__ldg(cf + static_cast<size_t>(kOff + slot) * a.K)); };
#include "generated/poly_lm5_forward.inc"
#pragma unroll
            for (int n = 0; n < NB; ++n)
                if (live[n]) a.M[(static_cast<size_t>(node[n]) * NOUT + 5) * a.K + k] = total.v[n];
        }
        {
            constexpr int kOff = kCanonPolyOffset[6];
            auto C = [&](int slot) { return T(__ldg(cf + static_cast<size_t>(kOff + slot) * a.K)); };
#include "generated/poly_lm6_forward.inc"
#pragma unroll
            for (int n = 0; n < NB; ++n)
                if (live[n]) a.M[(static_cast<size_t>(node[n]) * NOUT + 6) * a.K + k] = total.v[n];
        }
        {
            constexpr int kOff = kCanonPolyOffset[7];
            auto C = [&](int slot) { return T(__ldg(cf + static_cast<size_t>(kOff + slot) * a.K)); };
#include "generated/poly_lm7_forward.inc"
#pragma unroll
            for (int n = 0; n < NB; ++n)
                if (live[n]) a.M[(static_cast<size_t>(node[n]) * NOUT + 7) * a.K + k] = total.v[n];
        }
        {
            constexpr int kOff = kCanonPolyOffset[8];
            auto C = [&](int slot) { return T(__ldg(cf + static_cast<size_t>(kOff + slot) * a.K)); };
#include "generated/poly_lm8_forward.inc"
#pragma unroll
            for (int n = 0; n < NB; ++n)
                if (live[n]) a.M[(static_cast<size_t>(node[n]) * NOUT + 8) * a.K + k] = total.v[n];
        }
    }
}

template <typename S, int NOUT, int NB>
__global__ void __launch_bounds__(128) poly_fixed_reverse_kernel(const PolyArgs<S> a) {
    using T = PolyVec<S, NB>;
    // flat index -> (element type, group of NB nodes of that type, channel); groups of all types are numbered consecutively
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    int g = static_cast<int>(idx / a.K);
    const int k = static_cast<int>(idx - static_cast<long long>(g) * a.K);
    int type = 0, seg_begin = 0, count = 0;
    for (; type < a.num_types; ++type) {
        seg_begin = a.type_seg[type];
        count = a.type_seg[type + 1] - seg_begin;
        const int groups = (count + NB - 1) / NB;
        if (g < groups) break;
        g -= groups;
    }
    if (type == a.num_types) return;
    int node[NB];
    bool live[NB];
#pragma unroll
    for (int n = 0; n < NB; ++n) {
        const int jn = g * NB + n;
        live[n] = jn < count;
        node[n] = a.perm[seg_begin + (live[n] ? jn : count - 1)];   // an empty slot repeats the last node; its results are dropped
    }
    const S* cf = a.coef + static_cast<size_t>(type) * a.num_mono * a.K + k;
    T A[kNumLm], G[kNumLm];
#pragma unroll
    for (int q = 0; q < kNumLm; ++q) {
#pragma unroll
        for (int n = 0; n < NB; ++n) A[q].v[n] = a.A[(static_cast<size_t>(node[n]) * kNumLm + q) * a.K + k];
        G[q] = T(S(0));
    }
    {
        {
            constexpr int kOff = kCanonPolyOffset[0];
            auto C = [&](int slot) { return T(__ldg(cf + static_cast<size_t>(kOff + slot) * a.K)); };
            T seed;
#pragma unroll
            for (int n = 0; n < NB; ++n) seed.v[n] = a.M_adj[(static_cast<size_t>(node[n]) * NOUT + 0) * a.K + k];
#include "generated/poly_lm0_reverse.inc"
        }
    }
    if constexpr (NOUT > 1) {
        {
            constexpr int kOff = kCanonPolyOffset[1];
            auto C = [&](int slot) { return T(__ldg(cf + static_cast<size_t>(kOff + slot) * a.K)); };
            T seed;
#pragma unroll
            for (int n = 0; n < NB; ++n) seed.v[n] = a.M_adj[(static_cast<size_t>(node[n]) * NOUT + 1) * a.K + k];
#include "generated/poly_lm1_reverse.inc"
        }
        {
            constexpr int kOff = kCanonPolyOffset[2];
            auto C = [&](int slot) { return T(__ldg(cf + static_cast<size_t>(kOff + slot) * a.K)); };
            T seed;
#pragma unroll
            for (int n = 0; n < NB; ++n) seed.v[n] = a.M_adj[(static_cast<size_t>(node[n]) * NOUT + 2) * a.K + k];
#include "generated/poly_lm2_reverse.inc"
        }
        {
            constexpr int kOff = kCanonPolyOffset[3];
            auto C = [&](int slot) { return T(__ldg(cf + static_cast<size_t>(kOff + slot) * a.K)); };
            T seed;
#pragma unroll
            for (int n = 0; n < NB; ++n) seed.v[n] = a.M_adj[(static_cast<size_t>(node[n]) * NOUT + 3) * a.K + k];
#include "generated/poly_lm3_reverse.inc"
        }
    }
    if constexpr (NOUT > 4) {
        {
            constexpr int kOff = kCanonPolyOffset[4];
            auto C = [&](int slot) { return T(__ldg(cf + static_cast<size_t>(kOff + slot) * a.K)); };
            T seed;
#pragma unroll
            for (int n = 0; n < NB; ++n) seed.v[n] = a.M_adj[(static_cast<size_t>(node[n]) * NOUT + 4) * a.K + k];
#include "generated/poly_lm4_reverse.inc"
        }
        {
            constexpr int kOff = kCanonPolyOffset[5];
            auto C = [&](int slot) { return T(__ldg(cf + static_cast<size_t>(kOff + slot) * a.K)); };
            T seed;
#pragma unroll
            for (int n = 0; n < NB; ++n) seed.v[n] = a.M_adj[(static_cast<size_t>(node[n]) * NOUT + 5) * a.K + k];
#include "generated/poly_lm5_reverse.inc"
        }
        {
            constexpr int kOff = kCanonPolyOffset[6];
            auto C = [&](int slot) { return T(__ldg(cf + static_cast<size_t>(kOff + slot) * a.K)); };
            T seed;
#pragma unroll
            for (int n = 0; n < NB; ++n) seed.v[n] = a.M_adj[(static_cast<size_t>(node[n]) * NOUT + 6) * a.K + k];
#include "generated/poly_lm6_reverse.inc"
        }
        {
            constexpr int kOff = kCanonPolyOffset[7];
            auto C = [&](int slot) { return T(__ldg(cf + static_cast<size_t>(kOff + slot) * a.K)); };
            T seed;
#pragma unroll
            for (int n = 0; n < NB; ++n) seed.v[n] = a.M_adj[(static_cast<size_t>(node[n]) * NOUT + 7) * a.K + k];
#include "generated/poly_lm7_reverse.inc"
        }
        {
            constexpr int kOff = kCanonPolyOffset[8];
            auto C = [&](int slot) { return T(__ldg(cf + static_cast<size_t>(kOff + slot) * a.K)); };
            T seed;
#pragma unroll
            for (int n = 0; n < NB; ++n) seed.v[n] = a.M_adj[(static_cast<size_t>(node[n]) * NOUT + 8) * a.K + k];
#include "generated/poly_lm8_reverse.inc"
        }
    }
#pragma unroll
    for (int q = 0; q < kNumLm; ++q)
#pragma unroll
        for (int n = 0; n < NB; ++n)
            if (live[n]) a.A_adj[(static_cast<size_t>(node[n]) * kNumLm + q) * a.K + k] = G[q].v[n];
}

// =============================================================================================
// Channel-mixing linears as row-gathered GEMMs: C[row, :] (+)= A[row, :] . B  (or . B^T).
// A row of a problem is addressed as (node, sub): node = perm ? perm[seg_begin + r / sub_count]
// : r / sub_count, sub = r % sub_count, at A + node*a_node_stride + a_off + sub*a_sub_stride.
// One problem list entry per (element type, degree l) block; blockIdx.z selects the problem.
// Covers the dgemm/dgemv calls of compute_A0/H1/A1/H2 and their reverses (mace.cpp:184-198,
// 406-420, 623-637, 804-830 and :215-229, 434-448, 659-674, 846-872).
// =============================================================================================
template <typename T>
struct GemmProblem {
    const T* A; T* C; const T* B;
    const int* perm;         // optional node permutation (nodes sorted by element type)
    const int* seg;          // optional device array of segment offsets into perm
    int seg_index;           // this problem covers perm[seg[seg_index] .. seg[seg_index + 1])
    int num_nodes;           // used when seg == nullptr
    int sub_count;           // rows per node
    long long a_node_stride, a_off, a_sub_stride;
    long long c_node_stride, c_off, c_sub_stride;
    int Kd, Nc;              // inner dimension, output columns
    int ldb;                 // leading dimension of B
    int transB;              // 0: B is [Kd][Nc]; 1: B is [Nc][Kd] and used transposed
    int accumulate;          // 0: C = A.B ; 1: C += A.B
    const T* B_image;        // float32 tcgen05 path: B as pre-split, pre-swizzled operand tiles (gemm_tcgen05.cuh)
};

constexpr int kGemmBM = 64, kGemmBN = 64, kGemmBK = 16, kGemmThreads = 128;

// Tensor-core fragments. float64 uses the DMMA instruction mma.sync.m8n8k4 (sm_100a has no 5th-generation
// tensor-core kind for float64); float32 uses TF32 mma.sync.m16n8k8 with the operands split into a TF32 head
// and a TF32 remainder and three products per tile (head*head + head*rem + rem*head), which keeps float32-level
// accuracy for the 1e-4 energy gate while running on the tensor pipe.
__device__ __forceinline__ void dmma_m8n8k4(double& c0, double& c1, double a, double b) {
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};" : "+d"(c0), "+d"(c1) : "d"(a), "d"(b));
}
__device__ __forceinline__ unsigned to_tf32(float x) {
    unsigned r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ void mma_tf32_m16n8k8(float (&c)[4], const unsigned (&a)[4], const unsigned (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <typename T> struct GemmSmem;
template <> struct GemmSmem<double> { static constexpr int SA = kGemmBK + 4, SB = kGemmBN + 4; };   // conflict-free fragment reads
template <> struct GemmSmem<float> { static constexpr int SA = kGemmBK + 4, SB = kGemmBN + 8; };

// Warp tile 32 x 32 of the 64 x 64 CTA tile; accumulators and the k-loop body per precision.
template <typename T> struct WarpTile;
template <>
struct WarpTile<double> {
    double c[4][4][2];
    __device__ __forceinline__ void zero() {
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) c[i][j][0] = c[i][j][1] = 0.0;
    }
    __device__ __forceinline__ void step(const double* As, const double* Bs, int wm, int wn, int lane) {
        constexpr int SA = GemmSmem<double>::SA, SB = GemmSmem<double>::SB;
#pragma unroll
        for (int kk = 0; kk < kGemmBK; kk += 4) {
            double a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[(wm * 32 + i * 8 + (lane >> 2)) * SA + kk + (lane & 3)];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[(kk + (lane & 3)) * SB + wn * 32 + j * 8 + (lane >> 2)];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) dmma_m8n8k4(c[i][j][0], c[i][j][1], a[i], b[j]);
        }
    }
    template <typename F>
    __device__ __forceinline__ void for_each(int wm, int wn, int lane, F&& f) const {
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) f(wm * 32 + i * 8 + (lane >> 2), wn * 32 + j * 8 + 2 * (lane & 3) + e, c[i][j][e]);
    }
};
template <>
struct WarpTile<float> {
    float c[2][4][4];
    __device__ __forceinline__ void zero() {
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) c[i][j][e] = 0.f;
    }
    __device__ __forceinline__ void step(const float* As, const float* Bs, int wm, int wn, int lane) {
        constexpr int SA = GemmSmem<float>::SA, SB = GemmSmem<float>::SB;
#pragma unroll
        for (int kk = 0; kk < kGemmBK; kk += 8) {
            unsigned ah[2][4], al[2][4], bh[4][2], bl[4][2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int r = wm * 32 + i * 16 + (lane >> 2), cidx = kk + (lane & 3);
                const float v[4] = {As[r * SA + cidx], As[(r + 8) * SA + cidx], As[r * SA + cidx + 4], As[(r + 8) * SA + cidx + 4]};
#pragma unroll
                for (int e = 0; e < 4; ++e) { ah[i][e] = to_tf32(v[e]); al[i][e] = to_tf32(v[e] - __uint_as_float(ah[i][e])); }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int n = wn * 32 + j * 8 + (lane >> 2);
                const float v[2] = {Bs[(kk + (lane & 3)) * SB + n], Bs[(kk + 4 + (lane & 3)) * SB + n]};
#pragma unroll
                for (int e = 0; e < 2; ++e) { bh[j][e] = to_tf32(v[e]); bl[j][e] = to_tf32(v[e] - __uint_as_float(bh[j][e])); }
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    mma_tf32_m16n8k8(c[i][j], al[i], bh[j]);
                    mma_tf32_m16n8k8(c[i][j], ah[i], bl[j]);
                    mma_tf32_m16n8k8(c[i][j], ah[i], bh[j]);
                }
        }
    }
    template <typename F>
    __device__ __forceinline__ void for_each(int wm, int wn, int lane, F&& f) const {
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    f(wm * 32 + i * 16 + (lane >> 2) + (e >> 1) * 8, wn * 32 + j * 8 + 2 * (lane & 3) + (e & 1), c[i][j][e]);
    }
};

template <typename T>
__global__ void __launch_bounds__(kGemmThreads) gemm_rows_kernel(const GemmProblem<T>* __restrict__ problems) {
    const GemmProblem<T> pb = problems[blockIdx.z];
    int node_begin = 0, node_count = pb.num_nodes;
    if (pb.seg) { node_begin = pb.seg[pb.seg_index]; node_count = pb.seg[pb.seg_index + 1] - node_begin; }
    const long long M = static_cast<long long>(node_count) * pb.sub_count;
    const long long row0 = static_cast<long long>(blockIdx.x) * kGemmBM;
    const int col0 = blockIdx.y * kGemmBN;
    if (row0 >= M || col0 >= pb.Nc) return;

    constexpr int SA = GemmSmem<T>::SA, SB = GemmSmem<T>::SB;
    __shared__ T As[kGemmBM * SA];
    __shared__ T Bs[kGemmBK * SB];
    __shared__ long long a_base[kGemmBM];
    __shared__ long long c_base[kGemmBM];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp >> 1, wn = warp & 1;
    if (tid < kGemmBM) {
        const long long r = row0 + tid;
        if (r < M) {
            const long long n = r / pb.sub_count;
            const int sub = static_cast<int>(r - n * pb.sub_count);
            const long long node = pb.perm ? pb.perm[node_begin + n] : (node_begin + n);
            a_base[tid] = node * pb.a_node_stride + pb.a_off + sub * pb.a_sub_stride;
            c_base[tid] = node * pb.c_node_stride + pb.c_off + sub * pb.c_sub_stride;
        } else {
            a_base[tid] = -1;
            c_base[tid] = -1;
        }
    }
    __syncthreads();

    constexpr int kPer = kGemmBM * kGemmBK / kGemmThreads;   // 8 elements of each tile per thread
    T ra[kPer], rb[kPer];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int it = 0; it < kPer; ++it) {
            const int lin = tid + it * kGemmThreads;
            const int rr = lin >> 4, kk = lin & 15;
            ra[it] = (a_base[rr] >= 0 && k0 + kk < pb.Kd) ? pb.A[a_base[rr] + k0 + kk] : T(0);
            if (!pb.transB) {
                const int kb = lin >> 6, cc = lin & 63;
                rb[it] = (k0 + kb < pb.Kd && col0 + cc < pb.Nc) ? pb.B[static_cast<size_t>(k0 + kb) * pb.ldb + col0 + cc] : T(0);
            } else {
                const int cc = lin >> 4, kb = lin & 15;
                rb[it] = (k0 + kb < pb.Kd && col0 + cc < pb.Nc) ? pb.B[static_cast<size_t>(col0 + cc) * pb.ldb + k0 + kb] : T(0);
            }
        }
    };
    auto stash = [&]() {
#pragma unroll
        for (int it = 0; it < kPer; ++it) {
            const int lin = tid + it * kGemmThreads;
            As[(lin >> 4) * SA + (lin & 15)] = ra[it];
            if (!pb.transB) Bs[(lin >> 6) * SB + (lin & 63)] = rb[it];
            else Bs[(lin & 15) * SB + (lin >> 4)] = rb[it];
        }
    };

    WarpTile<T> acc;
    acc.zero();
    fetch(0);
    for (int k0 = 0; k0 < pb.Kd; k0 += kGemmBK) {
        stash();
        __syncthreads();
        if (k0 + kGemmBK < pb.Kd) fetch(k0 + kGemmBK);     // next tile's global loads overlap the tensor-core work
        acc.step(As, Bs, wm, wn, lane);
        __syncthreads();
    }
    acc.for_each(wm, wn, lane, [&](int r, int cidx, T v) {
        const long long cb = c_base[r];
        const int col = col0 + cidx;
        if (cb >= 0 && col < pb.Nc) {
            T* dst = pb.C + cb + col;
            *dst = pb.accumulate ? (*dst + v) : v;
        }
    });
}

// float64 variant with asynchronous tile loads: the 64 x 16 tile of gathered A rows and the 16 x 64 tile of B go from
// global to shared memory with 16-byte cp.async copies (no staging registers), two stages deep, so the copies of tile
// t + 1 run while the DMMA instructions work on tile t and there is one barrier pair per tile instead of a
// load - store - barrier sequence. Needs 16-byte aligned rows (even strides and offsets, even leading dimension); the
// launch code falls back to gemm_rows_kernel otherwise. Out-of-range rows, columns and k values are zero-filled by the
// copy's source-size operand.
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem)), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

static __global__ void __launch_bounds__(kGemmThreads) gemm_rows_f64_async_kernel(const GemmProblem<double>* __restrict__ problems) {
    const GemmProblem<double> pb = problems[blockIdx.z];
    int node_begin = 0, node_count = pb.num_nodes;
    if (pb.seg) { node_begin = pb.seg[pb.seg_index]; node_count = pb.seg[pb.seg_index + 1] - node_begin; }
    const long long M = static_cast<long long>(node_count) * pb.sub_count;
    const long long row0 = static_cast<long long>(blockIdx.x) * kGemmBM;
    const int col0 = blockIdx.y * kGemmBN;
    if (row0 >= M || col0 >= pb.Nc) return;

    constexpr int SA = GemmSmem<double>::SA, SB = GemmSmem<double>::SB;      // 20 and 68 doubles: rows start on 16-byte boundaries
    constexpr int kBTile = kGemmBK * SB > kGemmBN * SA ? kGemmBK * SB : kGemmBN * SA;
    __shared__ __align__(16) double As[2][kGemmBM * SA];
    __shared__ __align__(16) double Bs[2][kBTile];          // [k][n] rows of SB, or for transposed B [n][k] rows of SA
    __shared__ long long a_base[kGemmBM];
    __shared__ long long c_base[kGemmBM];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp >> 1, wn = warp & 1;
    if (tid < kGemmBM) {
        const long long r = row0 + tid;
        if (r < M) {
            const long long n = r / pb.sub_count;
            const int sub = static_cast<int>(r - n * pb.sub_count);
            const long long node = pb.perm ? pb.perm[node_begin + n] : (node_begin + n);
            a_base[tid] = node * pb.a_node_stride + pb.a_off + sub * pb.a_sub_stride;
            c_base[tid] = node * pb.c_node_stride + pb.c_off + sub * pb.c_sub_stride;
        } else {
            a_base[tid] = -1;
            c_base[tid] = -1;
        }
    }
    __syncthreads();

    auto issue = [&](int stage, int k0) {
        // A: 64 rows x 8 chunks of two doubles; B: 16 x 32 chunks (or 64 x 8 for transposed B): 4 + 4 chunks per thread
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int lin = tid + it * kGemmThreads;
            const int rr = lin >> 3, kk = (lin & 7) * 2;
            const long long ab = a_base[rr];
            const int left = pb.Kd - (k0 + kk);
            const int bytes = ab >= 0 ? (left >= 2 ? 16 : (left == 1 ? 8 : 0)) : 0;
            cp_async16(&As[stage][rr * SA + kk], pb.A + (bytes ? ab + k0 + kk : 0), bytes);
        }
        if (!pb.transB) {
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                const int lin = tid + it * kGemmThreads;
                const int kb = lin >> 5, cc = (lin & 31) * 2;
                const int left = pb.Nc - (col0 + cc);
                const int bytes = (k0 + kb < pb.Kd) ? (left >= 2 ? 16 : (left == 1 ? 8 : 0)) : 0;
                cp_async16(&Bs[stage][kb * SB + cc], pb.B + (bytes ? static_cast<size_t>(k0 + kb) * pb.ldb + col0 + cc : 0), bytes);
            }
        } else {
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                const int lin = tid + it * kGemmThreads;
                const int cc = lin >> 3, kb = (lin & 7) * 2;
                const int left = pb.Kd - (k0 + kb);
                const int bytes = (col0 + cc < pb.Nc) ? (left >= 2 ? 16 : (left == 1 ? 8 : 0)) : 0;
                cp_async16(&Bs[stage][cc * SA + kb], pb.B + (bytes ? static_cast<size_t>(col0 + cc) * pb.ldb + k0 + kb : 0), bytes);
            }
        }
        cp_async_commit();
    };

    double c[4][4][2];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) c[i][j][0] = c[i][j][1] = 0.0;
    const int num_tiles = (pb.Kd + kGemmBK - 1) / kGemmBK;
    issue(0, 0);
    for (int t = 0; t < num_tiles; ++t) {
        const int stage = t & 1;
        if (t + 1 < num_tiles) { issue(stage ^ 1, (t + 1) * kGemmBK); cp_async_wait<1>(); }
        else cp_async_wait<0>();
        __syncthreads();
        const double* Asm = As[stage];
        const double* Bsm = Bs[stage];
#pragma unroll
        for (int kk = 0; kk < kGemmBK; kk += 4) {
            double a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = Asm[(wm * 32 + i * 8 + (lane >> 2)) * SA + kk + (lane & 3)];
            if (!pb.transB) {
#pragma unroll
                for (int j = 0; j < 4; ++j) b[j] = Bsm[(kk + (lane & 3)) * SB + wn * 32 + j * 8 + (lane >> 2)];
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) b[j] = Bsm[(wn * 32 + j * 8 + (lane >> 2)) * SA + kk + (lane & 3)];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) dmma_m8n8k4(c[i][j][0], c[i][j][1], a[i], b[j]);
        }
        __syncthreads();      // this stage is refilled by the copies issued in the next iteration
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int r = wm * 32 + i * 8 + (lane >> 2), cidx = wn * 32 + j * 8 + 2 * (lane & 3) + e;
                const long long cb = c_base[r];
                const int col = col0 + cidx;
                if (cb >= 0 && col < pb.Nc) {
                    double* dst = pb.C + cb + col;
                    *dst = pb.accumulate ? (*dst + c[i][j][e]) : c[i][j][e];
                }
            }
}

// =============================================================================================
// Readouts (MACE::compute_readouts, mace.cpp:876-903 with MultilayerPerceptron::evaluate_gradient,
// multilayer_perceptron.cpp:76-150, hidden width 16): one warp per node.
//   E_i += E0[a] + w1 . H1[i,0,:] + w2 . (s * silu(W1 H2[i]))
//   H1_adj[i,0,:] = w1 ;  H2_adj[i,:] = W1^T (w2 * s * silu'(W1 H2[i]))
// H1_adj must have been zero-filled by the caller (the reference zero-fills it here).
// =============================================================================================
template <typename T>
struct ReadoutArgs {
    int N, K, nLM;
    const int* node_types;
    const double* E0;
    const T* ro1; const T* W1; const T* w2; T scale;
    const T* H1; const T* H2;
    double* node_energies;
    T* H1_adj; T* H2_adj;
    // three-block models: linear readout of the middle block's scalar features (null otherwise)
    const T* ro_m; const T* Hm; T* Hm_adj;
};

template <typename T>
__global__ void readout_kernel(const ReadoutArgs<T> a) {
    const int lane = threadIdx.x & 31;
    const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int warps_total = (gridDim.x * blockDim.x) >> 5;
    for (int i = warp_global; i < a.N; i += warps_total) {
        const T* h1 = a.H1 + static_cast<size_t>(i) * a.nLM * a.K;
        const T* h2 = a.H2 + static_cast<size_t>(i) * a.K;
        T lin = 0;
        T z[16];
#pragma unroll
        for (int h = 0; h < 16; ++h) z[h] = 0;
        for (int k = lane; k < a.K; k += 32) {
            lin += a.ro1[k] * h1[k];
            a.H1_adj[static_cast<size_t>(i) * a.nLM * a.K + k] = a.ro1[k];
            if (a.ro_m) {
                lin += a.ro_m[k] * a.Hm[static_cast<size_t>(i) * a.nLM * a.K + k];
                a.Hm_adj[static_cast<size_t>(i) * a.nLM * a.K + k] = a.ro_m[k];
            }
            const T v = h2[k];
#pragma unroll
            for (int h = 0; h < 16; ++h) z[h] += a.W1[h * a.K + k] * v;
        }
        lin = warp_sum(lin);
        T e2 = 0;
        T g[16];
#pragma unroll
        for (int h = 0; h < 16; ++h) {
            const T zz = warp_sum(z[h]);
            const T sig = T(1) / (T(1) + exp(-zz));
            e2 += a.w2[h] * (a.scale * zz * sig);
            g[h] = a.w2[h] * (a.scale * sig + a.scale * zz * sig * (T(1) - sig));
        }
        if (lane == 0) a.node_energies[i] += a.E0[a.node_types[i]] + double(lin) + double(e2);
        for (int k = lane; k < a.K; k += 32) {
            T s = 0;
#pragma unroll
            for (int h = 0; h < 16; ++h) s += g[h] * a.W1[h * a.K + k];
            a.H2_adj[static_cast<size_t>(i) * a.K + k] = s;
        }
    }
}

// =============================================================================================
// ZBL pair repulsion (ZBL::compute_ZBL, zbl.cpp:96-125 with compute / compute_gradient / envelope :22-94):
// screened Coulomb term times a polynomial envelope that vanishes at the sum of the covalent radii. Half of each
// pair energy goes to the receiver's node energy, the radial derivative to the edge's partial force. One thread
// per node walks its row, so the energy sum needs no atomics. Always float64.
// =============================================================================================
struct ZblParams {
    double a_exp, a_prefactor, c[4];
    int p;
    const double* covalent_radii;   // indexed by atomic number
    const int* atomic_numbers;      // per model type
};

static __global__ void zbl_kernel(int N, const int* __restrict__ node_types, const long long* __restrict__ first_neigh,
                           const int* __restrict__ neigh_types, const double* __restrict__ xyz, const double* __restrict__ r,
                           ZblParams z, double* __restrict__ node_energies, double* __restrict__ node_forces) {
    const double ce[4] = {-3.2, -0.9423, -0.4028, -0.2016};     // screening exponents, zbl.hpp:49-52
    const double v_prefactor = 14.3996;                          // zbl.hpp:53
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < N; i += gridDim.x * blockDim.x) {
        const int Zi = z.atomic_numbers[node_types[i]];
        double e_sum = 0.0;
        for (long long e = first_neigh[i]; e < first_neigh[i + 1]; ++e) {
            const int Zj = z.atomic_numbers[neigh_types[e]];
            const double rr = r[e];
            const double r_max = z.covalent_radii[Zi] + z.covalent_radii[Zj];
            if (rr >= r_max) continue;                           // envelope and its gradient vanish (zbl.cpp:76,86)
            const double Zu = Zi, Zv = Zj;
            const double a = z.a_prefactor * 0.529 / (pow(Zu, z.a_exp) + pow(Zv, z.a_exp));
            const double roa = rr / a;
            double phi = 0.0, dphi = 0.0;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const double t = z.c[q] * exp(ce[q] * roa);
                phi += t;
                dphi += ce[q] * t;
            }
            dphi /= a;
            const double v = v_prefactor * Zu * Zv / rr * phi;
            const double dv = v_prefactor * Zu * Zv * (rr * dphi - phi) / (rr * rr);
            const double x = rr / r_max, p = z.p;
            const double env = 1.0 - ((p + 1.0) * (p + 2.0) / 2.0) * pow(x, p) + p * (p + 2.0) * pow(x, p + 1.0) - (p * (p + 1.0) / 2.0) * pow(x, p + 2.0);
            const double denv = (-((p + 1.0) * (p + 2.0) / 2.0) * p * pow(x, p - 1.0) + p * (p + 2.0) * (p + 1.0) * pow(x, p)
                                 - (p * (p + 1.0) / 2.0) * (p + 2.0) * pow(x, p + 1.0)) / r_max;
            e_sum += 0.5 * v * env;
            const double g = 0.5 * (v * denv + dv * env);
            node_forces[3 * e] -= xyz[3 * e] / rr * g;
            node_forces[3 * e + 1] -= xyz[3 * e + 1] / rr * g;
            node_forces[3 * e + 2] -= xyz[3 * e + 2] / rr * g;
        }
        node_energies[i] += e_sum;
    }
}

// =============================================================================================
// Density normalisation of a layer's A features (MACE::compute_A0_scaled / reverse_A0_scaled and the A1 twins,
// mace.cpp:273-346, 681-757): A[i] /= 1 + sum_j f_ab(r_ij) with one scalar cubic spline per element pair.
// One CTA per node. The reverse pass recomputes the factor, adds dE/dr of the factor to the edge forces and
// scales the adjoint.
// =============================================================================================
struct ScalarSplines {
    const double* coef;   // [pair][bin][4]
    double h;
    int bins, num_elements;
};

__device__ __forceinline__ void scalar_spline(const ScalarSplines& sp, int type_i, int type_j, double rr, double& f, double& d) {
    const int lo = type_i <= type_j ? type_i : type_j, hi = type_i <= type_j ? type_j : type_i;
    const int pair = lo * (2 * sp.num_elements - lo - 1) / 2 + hi;
    int bin = static_cast<int>(rr / sp.h);
    bin = bin < 0 ? 0 : (bin > sp.bins - 1 ? sp.bins - 1 : bin);
    const double x = rr - sp.h * bin;
    const double* c = sp.coef + (static_cast<size_t>(pair) * sp.bins + bin) * 4;
    f = c[0] + c[1] * x + c[2] * x * x + c[3] * x * x * x;
    d = c[1] + 2 * c[2] * x + 3 * c[3] * x * x;
}

__device__ __forceinline__ double block_sum(double v, double* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    double t = 0;
    for (int w = 0; w < nw; ++w) t += sh[w];
    return t;
}

template <typename T>
__global__ void density_scale_forward_kernel(int N, int K, const int* __restrict__ node_types, const long long* __restrict__ first_neigh,
                                             const int* __restrict__ neigh_types, const double* __restrict__ r, ScalarSplines sp,
                                             T* __restrict__ A) {
    __shared__ double sh[32];
    for (int i = blockIdx.x; i < N; i += gridDim.x) {
        const int ti = node_types[i];
        double part = 0;
        for (long long e = first_neigh[i] + threadIdx.x; e < first_neigh[i + 1]; e += blockDim.x) {
            double f, d;
            scalar_spline(sp, ti, neigh_types[e], r[e], f, d);
            part += f;
        }
        const double factor = 1.0 + block_sum(part, sh);
        T* row = A + static_cast<size_t>(i) * kNumLm * K;
        for (int c = threadIdx.x; c < kNumLm * K; c += blockDim.x) row[c] = static_cast<T>(double(row[c]) / factor);
    }
}

template <typename T>
__global__ void density_scale_reverse_kernel(int N, int K, const int* __restrict__ node_types, const long long* __restrict__ first_neigh,
                                             const int* __restrict__ neigh_types, const double* __restrict__ xyz, const double* __restrict__ r,
                                             ScalarSplines sp, const T* __restrict__ A, T* __restrict__ A_adj, double* __restrict__ node_forces) {
    __shared__ double sh[32];
    for (int i = blockIdx.x; i < N; i += gridDim.x) {
        const int ti = node_types[i];
        double part = 0;
        for (long long e = first_neigh[i] + threadIdx.x; e < first_neigh[i + 1]; e += blockDim.x) {
            double f, d;
            scalar_spline(sp, ti, neigh_types[e], r[e], f, d);
            part += f;
        }
        const double factor = 1.0 + block_sum(part, sh);
        const T* arow = A + static_cast<size_t>(i) * kNumLm * K;
        T* grow = A_adj + static_cast<size_t>(i) * kNumLm * K;
        double dot = 0;
        for (int c = threadIdx.x; c < kNumLm * K; c += blockDim.x) dot += double(grow[c]) * double(arow[c]);
        dot = block_sum(dot, sh);
        for (long long e = first_neigh[i] + threadIdx.x; e < first_neigh[i + 1]; e += blockDim.x) {
            double f, d;
            scalar_spline(sp, ti, neigh_types[e], r[e], f, d);
            const double g = dot / factor * d / r[e];
            node_forces[3 * e] += g * xyz[3 * e];
            node_forces[3 * e + 1] += g * xyz[3 * e + 1];
            node_forces[3 * e + 2] += g * xyz[3 * e + 2];
        }
        __syncthreads();
        for (int c = threadIdx.x; c < kNumLm * K; c += blockDim.x) grow[c] = static_cast<T>(double(grow[c]) / factor);
    }
}

// =============================================================================================
// Small helpers
// =============================================================================================
static __global__ void iota_kernel(int n, int* out) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) out[i] = i;
}

// offsets[v] = first position in the sorted key array with key >= v, for v = 0..num_values
static __global__ void segment_offsets_kernel(long long n, const int* __restrict__ sorted_keys, int num_values, long long* __restrict__ offsets) {
    for (int v = blockIdx.x * blockDim.x + threadIdx.x; v <= num_values; v += gridDim.x * blockDim.x) {
        long long lo = 0, hi = n;
        while (lo < hi) {
            const long long mid = (lo + hi) >> 1;
            if (sorted_keys[mid] < v) lo = mid + 1; else hi = mid;
        }
        offsets[v] = lo;
    }
}
static __global__ void segment_offsets_int_kernel(int n, const int* __restrict__ sorted_keys, int num_values, int* __restrict__ offsets) {
    for (int v = blockIdx.x * blockDim.x + threadIdx.x; v <= num_values; v += gridDim.x * blockDim.x) {
        int lo = 0, hi = n;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (sorted_keys[mid] < v) lo = mid + 1; else hi = mid;
        }
        offsets[v] = lo;
    }
}

template <typename S, typename D>
__global__ void convert_kernel(long long n, const S* __restrict__ src, D* __restrict__ dst) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x)
        dst[i] = static_cast<D>(src[i]);
}

// Per-atom forces from per-edge partial forces, without atomics:
//   f[i] = - sum_{e in row i} nf[e] + sum_{e in in_edges(i)} nf[e]
// (pair_symmetrix/pair_symmetrix_mace.cpp:334-347; symmetrix_calc.py:93-97)
// One warp per atom: lane l takes the edges l, l + 32, ... of the atom's own row and of its incoming list in order, and the
// lanes are combined by a fixed shuffle tree (same bits on every run).
static __global__ void atom_forces_kernel(int rows, int N, const long long* __restrict__ first_neigh, const long long* __restrict__ in_ptr,
                                   const int* __restrict__ in_edge, const double* __restrict__ nf, double* __restrict__ f) {
    const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int i = blockIdx.x * warps + (threadIdx.x >> 5); i < rows; i += gridDim.x * warps) {
        double fx = 0, fy = 0, fz = 0;
        if (i < N)
            for (long long e = first_neigh[i] + lane; e < first_neigh[i + 1]; e += 32) { fx -= nf[3 * e]; fy -= nf[3 * e + 1]; fz -= nf[3 * e + 2]; }
        for (long long n = in_ptr[i] + lane; n < in_ptr[i + 1]; n += 32) {
            const long long e = in_edge[n];
            fx += nf[3 * e]; fy += nf[3 * e + 1]; fz += nf[3 * e + 2];
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            fx += __shfl_down_sync(0xffffffffu, fx, off);
            fy += __shfl_down_sync(0xffffffffu, fy, off);
            fz += __shfl_down_sync(0xffffffffu, fz, off);
        }
        if (lane == 0) { f[3 * i] = fx; f[3 * i + 1] = fy; f[3 * i + 2] = fz; }
    }
}

// ---------------------------------------------------------------------------------------------
// Halo rows of a decomposed run (what the reference's pair style does in pack_forward_comm / unpack_forward_comm /
// pack_reverse_comm / unpack_reverse_comm, pair_symmetrix/pair_symmetrix_mace.cpp:194-238, and as device kernels in
// pair_symmetrix_mace_kokkos.cpp:240-290, 351-367). Rows of `width` values, one thread per value.
//   gather:       buf[m, :]        = array[rows[m], :]
//   scatter:      array[rows[m], :] = buf[m, :]
//   scatter_add:  array[row, :]   += sum of buf[m, :] over the positions m with rows[m] == row, in ascending m
// The reference adds with atomics (order of the additions undefined); here the positions are grouped by row with a
// stable sort (`sorted_rows`, `sorted_pos`) and one thread adds a row's contributions in list order, so two runs give
// the same bits even when a row occurs several times in the list (an atom that is a ghost of the same peer twice).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void rows_gather_kernel(const T* __restrict__ array, int width, const int* __restrict__ rows, long long total, T* __restrict__ buf) {
    for (long long t = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; t < total; t += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long m = t / width;
        const int c = static_cast<int>(t - m * width);
        buf[t] = array[static_cast<size_t>(rows[m]) * width + c];
    }
}
template <typename T>
__global__ void rows_scatter_kernel(T* __restrict__ array, int width, const int* __restrict__ rows, long long total, const T* __restrict__ buf) {
    for (long long t = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; t < total; t += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long m = t / width;
        const int c = static_cast<int>(t - m * width);
        array[static_cast<size_t>(rows[m]) * width + c] = buf[t];
    }
}
template <typename T>
__global__ void rows_scatter_add_kernel(T* __restrict__ array, int width, const int* __restrict__ sorted_rows, const int* __restrict__ sorted_pos,
                                        int n, const T* __restrict__ buf) {
    const long long total = static_cast<long long>(n) * width;
    for (long long t = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; t < total; t += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int s = static_cast<int>(t / width);
        const int c = static_cast<int>(t - static_cast<long long>(s) * width);
        const int row = sorted_rows[s];
        if (s > 0 && sorted_rows[s - 1] == row) continue;        // not the first list position of this row
        T acc = array[static_cast<size_t>(row) * width + c];
        for (int q = s; q < n && sorted_rows[q] == row; ++q) acc += buf[static_cast<size_t>(sorted_pos[q]) * width + c];
        array[static_cast<size_t>(row) * width + c] = acc;
    }
}

// Block-wise partial sums of {energy, virial xx yy zz xy xz yz}; partials[block][7].
// Virial convention of pair_symmetrix_mace.cpp:349-368.
static __global__ void energy_virial_partial_kernel(int N, long long E, const double* __restrict__ node_energies, const double* __restrict__ xyz,
                                             const double* __restrict__ nf, double* __restrict__ partials) {
    __shared__ double sh[7][256];
    double v[7] = {0, 0, 0, 0, 0, 0, 0};
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < N; i += stride) v[0] += node_energies[i];
    for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < E; e += stride) {
        const double x = xyz[3 * e], y = xyz[3 * e + 1], z = xyz[3 * e + 2];
        const double fx = nf[3 * e], fy = nf[3 * e + 1], fz = nf[3 * e + 2];
        v[1] += x * fx; v[2] += y * fy; v[3] += z * fz;
        v[4] += 0.5 * (x * fy + y * fx); v[5] += 0.5 * (x * fz + z * fx); v[6] += 0.5 * (y * fz + z * fy);
    }
    for (int c = 0; c < 7; ++c) sh[c][threadIdx.x] = v[c];
    __syncthreads();
    for (int s = blockDim.x >> 1; s > 0; s >>= 1) {
        if (threadIdx.x < s)
            for (int c = 0; c < 7; ++c) sh[c][threadIdx.x] += sh[c][threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x < 7) partials[blockIdx.x * 7 + threadIdx.x] = sh[threadIdx.x][0];
}
// One warp per component (launch with 7 warps): lane l adds the rows l, l + 32, ... in order, then the lanes are combined
// by a fixed shuffle tree, so the sum has the same bits on every run.
static __global__ void energy_virial_final_kernel(int num_blocks, const double* __restrict__ partials, double* __restrict__ out7) {
    const int comp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (comp >= 7) return;
    double s = 0;
    for (int b = lane; b < num_blocks; b += 32) s += partials[b * 7 + comp];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_down_sync(0xffffffffu, s, off);
    if (lane == 0) out7[comp] = s;
}

}  // namespace smx
