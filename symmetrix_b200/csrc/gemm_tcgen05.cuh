// float32 channel-mixing GEMMs on the 5th-generation tensor cores (tcgen05.mma, accumulator in tensor memory).
//
// Same problem list as gemm_rows_kernel (rows gathered through (node, sub-row) strides and the type-sorted
// permutation). One CTA of 128 threads owns a 128 x 128 output tile whose accumulator lives in 128 columns of
// TMEM; three CTAs are resident per SM (64 KB of operand tiles each), so the loads, tensor-core work and
// epilogues of different tiles overlap. float32 accuracy comes from the 3xTF32 split x = hi + lo
// (hi = x with the 13 low mantissa bits cleared): per 8-wide k step the tensor core runs lo*hi + hi*lo + hi*hi.
//
// The k dimension is walked in chunks of 32 floats (one 128-byte swizzle atom per row). Per chunk
//   * B (the weights) comes from an operand image prepared once per weight matrix by gemm_tc5_prepare_b_kernel:
//     per (128-column block, k chunk) a hi tile and a lo tile already in the K-major, 128-byte-swizzled
//     shared-memory layout, so one thread brings both in with one bulk asynchronous copy (TMA) on an mbarrier;
//   * A (the gathered rows) is read with 16-byte loads, split in registers and stored as two swizzled tiles;
//     the loads of chunk i + 1 are issued before the CTA waits for the tensor core to finish chunk i;
//   * one thread issues the 12 MMAs of the chunk and commits them to an mbarrier.
// Every wait is bounded: if an mbarrier does not flip within the spin budget the CTA records an error code, skips
// further tensor-core work, frees its TMEM and returns.
#pragma once

#include <cuda_runtime.h>

#include <cuda_fp16.h>

#include <cstdint>

#include "kernels.cuh"

namespace smx {

constexpr int kTc5BM = 128, kTc5BN = 128, kTc5BK = 32, kTc5Threads = 128;
constexpr int kTc5TileBytes = kTc5BM * kTc5BK * 4;                       // 16 KB per operand tile
constexpr int kTc5TileFloats = kTc5TileBytes / 4;
constexpr int kTc5SmemBytes = 4 * kTc5TileBytes + 1024;                  // A_hi, A_lo, B_hi, B_lo + slack for 1024-byte alignment
constexpr unsigned kTc5HiMask = 0xFFFFE000u;

// byte offset of the 16-byte group `c4` (4 floats) of row `row` in a K-major tile of 32 floats per row with the
// 128-byte swizzle: rows in groups of 8 (1024 bytes), 16-byte group index XOR-ed with the row index inside the group
__host__ __device__ __forceinline__ int tc5_swizzled_group(int row, int c4) {
    const int r8 = row & 7;
    return (row >> 3) * 1024 + r8 * 128 + ((c4 ^ r8) << 4);
}

// floats of the operand image of a [Kd] x [Nc] weight matrix: [column block][k chunk][hi, lo][tile]
inline size_t tc5_image_floats(int Kd, int Nc) {
    return static_cast<size_t>((Nc + kTc5BN - 1) / kTc5BN) * ((Kd + kTc5BK - 1) / kTc5BK) * 2 * kTc5TileFloats;
}

// One thread per (column block, k chunk, column n, 16-byte group): reads four weights, zero beyond the matrix,
// and writes the hi and lo values where the tensor core expects column n of the K-major B tile.
static __global__ void gemm_tc5_prepare_b_kernel(const float* __restrict__ B, int Kd, int Nc, int ldb, int transB, float* __restrict__ image) {
    const int k_chunks = (Kd + kTc5BK - 1) / kTc5BK, n_blocks = (Nc + kTc5BN - 1) / kTc5BN;
    const long long total = static_cast<long long>(n_blocks) * k_chunks * kTc5BN * (kTc5BK / 4);
    for (long long t = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; t < total; t += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int c4 = static_cast<int>(t & 7);
        const int n = static_cast<int>((t >> 3) & (kTc5BN - 1));
        const long long tile = t >> 10;                     // column block * k_chunks + k chunk
        const int kc = static_cast<int>(tile % k_chunks), nb = static_cast<int>(tile / k_chunks);
        float hi[4], lo[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int k = kc * kTc5BK + c4 * 4 + q, col = nb * kTc5BN + n;
            float v = 0.f;
            if (k < Kd && col < Nc) v = transB ? B[static_cast<size_t>(col) * ldb + k] : B[static_cast<size_t>(k) * ldb + col];
            hi[q] = __uint_as_float(__float_as_uint(v) & kTc5HiMask);
            lo[q] = v - hi[q];
        }
        float* base = image + static_cast<size_t>(tile) * 2 * kTc5TileFloats;
        const int off = tc5_swizzled_group(n, c4) >> 2;
        *reinterpret_cast<float4*>(base + off) = make_float4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<float4*>(base + kTc5TileFloats + off) = make_float4(lo[0], lo[1], lo[2], lo[3]);
    }
}

// shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t tc5_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);            // start address
    d |= static_cast<uint64_t>(1) << 16;                               // leading byte offset (unused for swizzled K-major)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;                       // stride byte offset: next 8-row group
    d |= static_cast<uint64_t>(1) << 46;                               // descriptor version
    d |= static_cast<uint64_t>(2) << 61;                               // layout: 128-byte swizzle
    return d;
}

// instruction descriptor: D = F32, A = B = TF32, both K-major, M = 128, N = 128
__device__ __forceinline__ uint32_t tc5_instr_desc() {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((kTc5BN >> 3) << 17) | ((kTc5BM >> 4) << 24);
}

__device__ __forceinline__ void tc5_mma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void tc5_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// `status[0]` receives a non-zero code if a bounded wait ran out (1: tensor core, 2: weight tile copy).
// `status[1]` is a test switch, zero in normal operation: when set, the first weight-tile wait of every CTA expects 16
// bytes more than the copy delivers and polls only `status[1]` times, so the wait runs out quickly and the error path
// (status word, TMEM release, host-side error) can be exercised without any fault.
// Every problem carries the operand image of its weight matrix in B_image.
static __global__ void __launch_bounds__(kTc5Threads) gemm_rows_tcgen05_kernel(const GemmProblem<float>* __restrict__ problems, int* __restrict__ status) {
    const GemmProblem<float> pb = problems[blockIdx.z];
    int node_begin = 0, node_count = pb.num_nodes;
    if (pb.seg) { node_begin = pb.seg[pb.seg_index]; node_count = pb.seg[pb.seg_index + 1] - node_begin; }
    const long long M = static_cast<long long>(node_count) * pb.sub_count;
    const long long row0 = static_cast<long long>(blockIdx.x) * kTc5BM;
    const int col0 = blockIdx.y * kTc5BN;
    if (row0 >= M || col0 >= pb.Nc || pb.Kd <= 0) return;

    extern __shared__ unsigned char tc5_smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc5_smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char* sA_hi = tiles;
    unsigned char* sA_lo = sA_hi + kTc5TileBytes;
    unsigned char* sB = sA_lo + kTc5TileBytes;                // B_hi then B_lo, contiguous as in the image
    __shared__ __align__(8) unsigned long long mma_bar, b_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ long long a_base[kTc5BM];
    __shared__ long long c_base[kTc5BM];
    __shared__ int failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    {
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
    if (tid == 0) {
        failed = 0;
        mbar_init(&mma_bar, 1);
        mbar_init(&b_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(kTc5BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_base_slot;
    const uint32_t idesc = tc5_instr_desc();
    const int expire_test = status[1];
    const unsigned spin_limit = expire_test > 0 ? static_cast<unsigned>(expire_test) : kMbarSpinLimit;

    const int num_chunks = (pb.Kd + kTc5BK - 1) / kTc5BK;
    const float* image = pb.B_image + static_cast<size_t>(blockIdx.y) * num_chunks * 2 * kTc5TileFloats;
    // 16-byte loads need rows that start on a 16-byte boundary and a k extent that is a multiple of 4 (true for
    // every problem the evaluator builds when K is a multiple of 4); otherwise the loads are scalar
    const bool vec_ok = (pb.Kd & 3) == 0 && ((pb.a_node_stride | pb.a_off | pb.a_sub_stride) & 3) == 0 &&
                        (reinterpret_cast<uintptr_t>(pb.A) & 15) == 0;

    float4 pre[8];
    auto load_chunk = [&](int ch) {
        const int k0 = ch * kTc5BK;
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int lin = tid + it * kTc5Threads;
            const int rr = lin >> 3, kk = k0 + ((lin & 7) << 2);
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            const long long ab = a_base[rr];
            if (ab >= 0) {
                if (vec_ok && kk + 3 < pb.Kd) {
                    v = *reinterpret_cast<const float4*>(pb.A + ab + kk);
                } else {
                    if (kk < pb.Kd) v.x = pb.A[ab + kk];
                    if (kk + 1 < pb.Kd) v.y = pb.A[ab + kk + 1];
                    if (kk + 2 < pb.Kd) v.z = pb.A[ab + kk + 2];
                    if (kk + 3 < pb.Kd) v.w = pb.A[ab + kk + 3];
                }
            }
            pre[it] = v;
        }
    };
    load_chunk(0);
    unsigned mma_par = 0, b_par = 0;
    for (int ch = 0; ch < num_chunks; ++ch) {
        // the MMAs of the previous chunk read the tiles: wait for them before overwriting
        if (ch > 0) {
            if (!*reinterpret_cast<volatile int*>(&failed) && !mbar_wait(&mma_bar, mma_par, spin_limit)) atomicMax(&failed, 1);
            mma_par ^= 1u;
        }
        __syncthreads();
        if (tid == 0 && !failed) {
            mbar_expect_tx(&b_bar, 2 * kTc5TileBytes + ((expire_test > 0 && ch == 0) ? 16 : 0));
            bulk_copy_g2s(sB, image + static_cast<size_t>(ch) * 2 * kTc5TileFloats, 2 * kTc5TileBytes, &b_bar);
        }
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int lin = tid + it * kTc5Threads;
            const int off = tc5_swizzled_group(lin >> 3, lin & 7);
            const float4 v = pre[it];
            float4 hi, lo;
            hi.x = __uint_as_float(__float_as_uint(v.x) & kTc5HiMask); lo.x = v.x - hi.x;
            hi.y = __uint_as_float(__float_as_uint(v.y) & kTc5HiMask); lo.y = v.y - hi.y;
            hi.z = __uint_as_float(__float_as_uint(v.z) & kTc5HiMask); lo.z = v.z - hi.z;
            hi.w = __uint_as_float(__float_as_uint(v.w) & kTc5HiMask); lo.w = v.w - hi.w;
            *reinterpret_cast<float4*>(sA_hi + off) = hi;
            *reinterpret_cast<float4*>(sA_lo + off) = lo;
        }
        if (ch + 1 < num_chunks) load_chunk(ch + 1);            // in flight while the tensor core works on this chunk
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic-proxy stores -> visible to the tensor core
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0 && !failed) {
            if (!mbar_wait(&b_bar, b_par, spin_limit)) {
                atomicMax(&failed, 2);
            } else {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_hi = smem_u32(sA_hi), a_lo = smem_u32(sA_lo), b_hi = smem_u32(sB), b_lo = smem_u32(sB + kTc5TileBytes);
#pragma unroll
                for (int ks = 0; ks < kTc5BK / 8; ++ks) {
                    const uint32_t adv = ks * 32;        // 8 TF32 values = 32 bytes inside the swizzle atom
                    const uint32_t first = (ch == 0 && ks == 0) ? 0u : 1u;
                    tc5_mma(tmem_d, tc5_smem_desc(a_lo + adv), tc5_smem_desc(b_hi + adv), idesc, first);
                    tc5_mma(tmem_d, tc5_smem_desc(a_hi + adv), tc5_smem_desc(b_lo + adv), idesc, 1u);
                    tc5_mma(tmem_d, tc5_smem_desc(a_hi + adv), tc5_smem_desc(b_hi + adv), idesc, 1u);
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&mma_bar)) : "memory");
            }
        }
        b_par ^= 1u;
    }
    __syncthreads();                                             // `failed` as thread 0 left it
    if (!*reinterpret_cast<volatile int*>(&failed) && !mbar_wait(&mma_bar, mma_par, spin_limit)) atomicMax(&failed, 1);
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (!failed) {
        // Epilogue. A thread holds one output row (its TMEM lane); writing rows straight from registers would make
        // every store instruction touch 32 different rows. The warp therefore passes its 32 x 128 block through the
        // (now idle) operand tiles, 16-byte groups XOR-swizzled by the row so that both the row-wise writes and the
        // column-wise reads are free of bank conflicts, and then stores whole 512-byte rows per instruction.
        float* stage = reinterpret_cast<float*>(tiles) + warp * (32 * kTc5BN);
#pragma unroll 1
        for (int cc = 0; cc < kTc5BN / 32; ++cc) {
            uint32_t v[32];
            tc5_ld32(tmem_d + (static_cast<uint32_t>(warp * 32) << 16) + cc * 32, v);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int g = cc * 8 + j;
                *reinterpret_cast<float4*>(stage + lane * kTc5BN + ((g ^ lane) << 2)) =
                    make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
            }
        }
        __syncwarp();
        const bool cvec = ((pb.c_node_stride | pb.c_off | pb.c_sub_stride) & 3) == 0 && (reinterpret_cast<uintptr_t>(pb.C) & 15) == 0;
        const int col = col0 + lane * 4;
#pragma unroll 4
        for (int r = 0; r < 32; ++r) {
            const long long cb = c_base[warp * 32 + r];
            if (cb < 0) continue;
            float4 o = *reinterpret_cast<const float4*>(stage + r * kTc5BN + ((lane ^ r) << 2));
            float* dst = pb.C + cb + col;
            if (cvec && col + 3 < pb.Nc) {
                if (pb.accumulate) {
                    const float4 old = *reinterpret_cast<const float4*>(dst);
                    o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4*>(dst) = o;
            } else {
                const float ov[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (col + q < pb.Nc) dst[q] = pb.accumulate ? (dst[q] + ov[q]) : ov[q];
            }
        }
    } else if (tid == 0) {
        atomicMax(status, failed);
        // a weight-tile copy that may still be in flight gets one more bounded wait before the CTA exits
        mbar_wait(&b_bar, b_par ^ 1u, spin_limit);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(kTc5BN) : "memory");
}

// =============================================================================================
// Tensor product (forward) of block 1 with the radial functions evaluated on the tensor cores inside the kernel.
//
// The edge kernels that read spline tables stream 4 coefficients per (edge, path, channel) from L2 -- 20 KB per edge in
// float32 for 10 paths x 128 channels -- and run at the speed of that stream. The radial functions are the outputs of
// a small network, R[e, (p, k)] = sum_j x[e, j] W[j, (p, k)] with x the hidden activations of the edge
// (radial_hidden_kernel, 64 values per edge), so per batch of 16 edges the P x 128 x 16 values are one small GEMM per path:
//     D_p[k, e] = sum_j A_p[k, j] B[e, j],   A_p = W[:, (p, :)]^T  (128 x 64, float16, resident in shared memory for the
//                                            whole kernel: P x 16 KB), B = x of the batch (16 x 64, float16)
// issued as tcgen05.mma (kind::f16, M = 128, N = 16, K = 16, float32 accumulation) by one thread, with the result in
// tensor memory: lane = channel, column = (path, edge). The thread that owns channel k reads its radial values with
// tcgen05.ld, so nothing but the 128 bytes of x per edge is streamed. float16 operands (11-bit significands) keep the
// radial values to about 1e-4 relative, inside the float32 gates.
//
// One CTA of 512 threads per SM (the operand tiles take 160 KB of shared memory): warp w works on the channels of TMEM
// quadrant w % 4 and, as member of group w / 4, on 4 of the 16 edges of a batch; the groups' partial sums over edges are
// added through shared memory when a receiver is finished. Batches are double-buffered (operand B, per-edge data and the
// 160 accumulator columns), so the tensor core works on batch b + 1 while the CUDA cores consume batch b; a CTA walks
// the batches of all its receivers as one sequence. Every mbarrier wait is bounded (status codes 5, 6).
// =============================================================================================
constexpr int kRnEdges = 16, kRnGroups = 4, kRnThreads = 512, kRnHidden = 64;
constexpr int kRnTileBytes = 128 * kRnHidden * 2;          // one path's weight tile, float16
constexpr int kRnBTileBytes = kRnEdges * kRnHidden * 2;

// byte offset of element (row, j) in a K-major tile of 64 float16 per row with the 128-byte swizzle
__host__ __device__ __forceinline__ int rn_swizzled(int row, int j) {
    return (row >> 3) * 1024 + (row & 7) * 128 + ((((j >> 3) ^ (row & 7)) & 7) << 4) + (j & 7) * 2;
}

// Weight tiles of the last layer: image[c][swizzled (k, j)] = half(w_last[j][c * K + k]), zero beyond K or the hidden width.
static __global__ void radial_prepare_tiles_kernel(const float* __restrict__ w_last, int hidden, int K, int P, unsigned char* __restrict__ image) {
    const int total = P * 128 * kRnHidden;
    for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < total; t += gridDim.x * blockDim.x) {
        const int j = t % kRnHidden, k = (t / kRnHidden) % 128, c = t / (kRnHidden * 128);
        const float v = (k < K && j < hidden) ? w_last[static_cast<size_t>(j) * P * K + c * K + k] : 0.f;
        *reinterpret_cast<__half*>(image + static_cast<size_t>(c) * kRnTileBytes + rn_swizzled(k, j)) = __float2half_rn(v);
    }
}

__device__ __forceinline__ uint32_t rn_instr_desc() {   // D = F32, A = B = F16, both K-major, M = 128, N = 16
    return (1u << 4) | (0u << 7) | (0u << 10) | ((kRnEdges >> 3) << 17) | ((128 >> 4) << 24);
}
__device__ __forceinline__ void rn_mma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, float (&v)[4]) {
    uint32_t r0, r1, r2, r3;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(r0), "+r"(r1), "+r"(r2), "+r"(r3)::"memory");
    v[0] = __uint_as_float(r0); v[1] = __uint_as_float(r1); v[2] = __uint_as_float(r2); v[3] = __uint_as_float(r3);
}

// Source of the hidden activations that fill operand B: arrays written by radial_hidden_kernel (x, dx: [num_edges][hidden]),
// or -- when `basis` is set -- the tabulated last hidden layer, cubic coefficients [pair][bin][hidden][4] on the grid of the
// radial splines, evaluated here per (edge, hidden unit) with the bin rule of the spline path (stage_edge).
struct RnHidden {
    const float* x; const float* dx;
    const float* basis;
    SplineMeta sm;
    int hidden;
};
__device__ __forceinline__ void rn_hidden_pair(const RnHidden& hd, const TPArgs<float>& a, int type_i, long long edge, int j0, bool want_dx,
                                               float2& v, float2& dv) {
    v = make_float2(0.f, 0.f); dv = make_float2(0.f, 0.f);
    if (hd.basis) {
        const double rr = a.r[edge];
        int bin = static_cast<int>(rr / hd.sm.h);
        bin = bin < 0 ? 0 : (bin > hd.sm.num_bins - 1 ? hd.sm.num_bins - 1 : bin);
        const float x = static_cast<float>(rr - hd.sm.h * bin);
        const int tj = a.neigh_types[edge];
        const int lo = type_i <= tj ? type_i : tj, hi = type_i <= tj ? tj : type_i;
        const int pair = lo * (2 * hd.sm.num_elements - lo - 1) / 2 + hi;
        const float4* row = reinterpret_cast<const float4*>(hd.basis) + (static_cast<size_t>(pair) * hd.sm.num_bins + bin) * hd.hidden;
        if (j0 < hd.hidden) {
            const float4 c = __ldg(row + j0);
            v.x = c.x + x * (c.y + x * (c.z + x * c.w));
            dv.x = c.y + x * (2.f * c.z + 3.f * x * c.w);
        }
        if (j0 + 1 < hd.hidden) {
            const float4 c = __ldg(row + j0 + 1);
            v.y = c.x + x * (c.y + x * (c.z + x * c.w));
            dv.y = c.y + x * (2.f * c.z + 3.f * x * c.w);
        }
    } else {
        const float* r0 = hd.x + static_cast<size_t>(edge) * hd.hidden;
        if (j0 < hd.hidden) v.x = r0[j0];
        if (j0 + 1 < hd.hidden) v.y = r0[j0 + 1];
        if (want_dx) {
            const float* r1 = hd.dx + static_cast<size_t>(edge) * hd.hidden;
            if (j0 < hd.hidden) dv.x = r1[j0];
            if (j0 + 1 < hd.hidden) dv.y = r1[j0 + 1];
        }
    }
}

// Starts the fetch of 4 accumulator columns; rn_ld_wait completes all fetches of the thread (the registers are operands of
// the wait so that no use of them is scheduled before it).
__device__ __forceinline__ void rn_ld4_issue(uint32_t taddr, uint32_t (&v)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(taddr) : "memory");
}
template <int P>
__device__ __forceinline__ void rn_ld_wait(uint32_t (&v)[P][4]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int p = 0; p < P; ++p) asm volatile("" : "+r"(v[p][0]), "+r"(v[p][1]), "+r"(v[p][2]), "+r"(v[p][3]) :: "memory");
}

struct RnEdge {             // per-edge, channel-independent data of the forward pass
    float Y[kNumLm];
    int j;                  // sender row
};

template <int LF>
struct RnSmem {
    static constexpr TPTable tp = make_tp_table(LF);
    static constexpr int kTiles = tp.P * kRnTileBytes;
    static constexpr int kB = 2 * kRnBTileBytes;                             // both B tiles start on 1024-byte boundaries
    static constexpr int kEdge = 2 * kRnEdges * static_cast<int>(sizeof(RnEdge));
    static constexpr int kXchg = 2 * tp.Q * 128 * 4;                         // two groups' partial sums
    static constexpr int kTotal = 1024 + kTiles + kB + kEdge + kXchg;
    static constexpr int kDCols = tp.P * kRnEdges;                           // accumulator columns per buffer
};
constexpr int rn_tmem_cols(int dcols) { int a = 32; while (a < 2 * dcols) a *= 2; return a; }

template <int LF>
__global__ void __launch_bounds__(kRnThreads, 1) tp_forward_rnet_kernel(const TPArgs<float> a, const unsigned char* __restrict__ tiles_image,
                                                                        const RnHidden hd) {
    using S = RnSmem<LF>;
    constexpr TPTable tp = make_tp_table(LF);
    constexpr int kDCols = S::kDCols, kCols = rn_tmem_cols(kDCols);
    static_assert(kCols <= 512, "accumulator columns of two batches must fit into tensor memory");
    extern __shared__ unsigned char rn_smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(rn_smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char* sA = base;
    unsigned char* sB = sA + S::kTiles;
    RnEdge* st = reinterpret_cast<RnEdge*>(sB + S::kB);
    float* xchg = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(st) + S::kEdge);
    __shared__ __align__(8) unsigned long long a_bar, mma_bar[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int group = warp >> 2, k = (warp & 3) * 32 + lane;      // channel = TMEM lane
    const bool active = k < a.K;
    if (tid == 0) {
        failed = 0;
        mbar_init(&a_bar, 1); mbar_init(&mma_bar[0], 1); mbar_init(&mma_bar[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(kCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_slot;
    const uint32_t my_taddr = tmem_d + (static_cast<uint32_t>((warp & 3) * 32) << 16) + 4 * group;
    if (tid == 0) {      // the weight tiles of all paths, once per CTA
        mbar_expect_tx(&a_bar, S::kTiles);
        for (int p = 0; p < tp.P; ++p) bulk_copy_g2s(sA + p * kRnTileBytes, tiles_image + static_cast<size_t>(p) * kRnTileBytes, kRnTileBytes, &a_bar);
    }
    bool tiles_ready = false;
    const uint32_t idesc = rn_instr_desc();
    unsigned mma_par[2] = {0u, 0u};

    // ---- the CTA's batches as one sequence: (receiver slot, first edge of the batch)
    struct Cursor { int slot; int i; int type_i; long long e0, e_end; };
    auto load_receiver = [&](Cursor& c) {          // positions `c` on the first batch of receiver slot c.slot (or past the end)
        if (c.slot < a.N) {
            c.i = a.order ? a.order[c.slot] : c.slot;
            c.type_i = a.node_types[c.i];
            c.e0 = a.first_neigh[c.i];
            c.e_end = a.first_neigh[c.i + 1];
        }
    };
    auto advance = [&](Cursor& c) {                // next batch; receivers without edges are batches with zero edges
        c.e0 += kRnEdges;
        if (c.e0 >= c.e_end) { c.slot += gridDim.x; load_receiver(c); }
    };
    // stage batch `c` into buffer `buf`: per-edge harmonics and sender row, and the B tile (hidden activations as float16)
    auto stage_batch = [&](const Cursor& c, int buf) {
        const int nb = static_cast<int>(c.e_end - c.e0 < kRnEdges ? c.e_end - c.e0 : kRnEdges);
        // the harmonics of the batch's edges: the first 16 lanes of the last warp (the first warp issues the tensor-core work)
        if (warp == kRnThreads / 32 - 1 && lane < kRnEdges) {
            RnEdge& s = st[buf * kRnEdges + lane];
            if (lane < nb) {
                const long long e = c.e0 + lane;
                const double rr = a.r[e], inv = 1.0 / rr;
                float dummy[3][kNumLm];
                real_sh3<float, false>(float(a.xyz[3 * e] * inv), float(a.xyz[3 * e + 1] * inv), float(a.xyz[3 * e + 2] * inv), float(inv), s.Y, dummy);
                s.j = a.neigh_indices[e];
            } else {
                s.j = 0;
            }
        }
        {   // 16 edges x 64 activations: two per thread
            const int e = tid >> 5, j0 = (tid & 31) * 2;
            float2 v = make_float2(0.f, 0.f), dv;
            if (e < nb) rn_hidden_pair(hd, a, c.type_i, c.e0 + e, j0, false, v, dv);
            *reinterpret_cast<__half2*>(sB + buf * kRnBTileBytes + rn_swizzled(e, j0)) = __floats2half2_rn(v.x, v.y);
        }
    };
    auto issue_mma = [&](int buf) {                // one thread: P x 4 MMAs into the accumulator columns of `buf`
        const uint32_t b_addr = smem_u32(sB + buf * kRnBTileBytes);
#pragma unroll 1
        for (int p = 0; p < tp.P; ++p) {
            const uint32_t a_addr = smem_u32(sA + p * kRnTileBytes);
#pragma unroll
            for (int ks = 0; ks < kRnHidden / 16; ++ks)
                rn_mma(tmem_d + buf * kDCols + p * kRnEdges, tc5_smem_desc(a_addr + ks * 32), tc5_smem_desc(b_addr + ks * 32), idesc, ks > 0 ? 1u : 0u);
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&mma_bar[buf])) : "memory");
    };

    Cursor cur{static_cast<int>(blockIdx.x), 0, 0, 0, 0};
    load_receiver(cur);
    float acc[tp.Q];
#pragma unroll
    for (int q = 0; q < tp.Q; ++q) acc[q] = 0.f;
    int buf = 0;
    if (cur.slot < a.N) {
        stage_batch(cur, 0);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            if (!mbar_wait(&a_bar, 0)) { atomicMax(&failed, 5); }
            else { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); issue_mma(0); }
        }
        tiles_ready = true;
    }
    while (cur.slot < a.N) {
        Cursor nxt = cur;
        advance(nxt);
        const bool have_next = nxt.slot < a.N;
        if (have_next) stage_batch(nxt, buf ^ 1);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (have_next && tid == 0 && !failed) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            issue_mma(buf ^ 1);
        }
        // ---- consume batch `cur` from buffer `buf`
        if (!*reinterpret_cast<volatile int*>(&failed) && !mbar_wait(&mma_bar[buf], mma_par[buf])) atomicMax(&failed, 6);
        mma_par[buf] ^= 1u;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int nb = static_cast<int>(cur.e_end - cur.e0 < kRnEdges ? cur.e_end - cur.e0 : kRnEdges);
        if (!*reinterpret_cast<volatile int*>(&failed)) {
            uint32_t Rq[tp.P][4];
#pragma unroll
            for (int p = 0; p < tp.P; ++p) rn_ld4_issue(my_taddr + buf * kDCols + p * kRnEdges, Rq[p]);
            // sender features of the group's four edges: all loads in flight before the first use
            float hq[4][tp.nLM];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const int e = 4 * group + t;
                const float* hrow = a.H + static_cast<size_t>(st[buf * kRnEdges + (e < nb ? e : 0)].j) * tp.nLM * a.K + k;
#pragma unroll
                for (int lm2 = 0; lm2 < tp.nLM; ++lm2) hq[t][lm2] = (e < nb && active) ? __ldg(hrow + static_cast<size_t>(lm2) * a.K) : 0.f;
            }
            rn_ld_wait<tp.P>(Rq);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const int e = 4 * group + t;
                if (e < nb && active) {
                    const RnEdge& s = st[buf * kRnEdges + e];
                    float h[tp.nLM], R[tp.P], Y[kNumLm];
#pragma unroll
                    for (int lm2 = 0; lm2 < tp.nLM; ++lm2) h[lm2] = hq[t][lm2];
#pragma unroll
                    for (int p = 0; p < tp.P; ++p) R[p] = __uint_as_float(Rq[p][t]);
#pragma unroll
                    for (int lm = 0; lm < kNumLm; ++lm) Y[lm] = s.Y[lm];
                    using T = float;
                    using ::fma;      // the generated code calls fma on plain floats (namespace smx has its own fma for node vectors)
                    if constexpr (LF == 0) {
#include "generated/tp_L0_forward.inc"
                    } else if constexpr (LF == 1) {
#include "generated/tp_L1_forward.inc"
                    } else {
#include "generated/tp_L2_forward.inc"
                    }
                }
            }
        }
        const bool receiver_done = !have_next || nxt.slot != cur.slot;
        if (receiver_done) {
            // add the four groups' partial sums: groups 2, 3 -> shared memory -> groups 0, 1; then group 1 -> group 0 -> HBM
            __syncthreads();
            if (group >= 2) {
#pragma unroll
                for (int q = 0; q < tp.Q; ++q) xchg[((group - 2) * tp.Q + q) * 128 + k] = acc[q];
            }
            __syncthreads();
            if (group < 2) {
#pragma unroll
                for (int q = 0; q < tp.Q; ++q) acc[q] += xchg[(group * tp.Q + q) * 128 + k];
            }
            __syncthreads();
            if (group == 1) {
#pragma unroll
                for (int q = 0; q < tp.Q; ++q) xchg[q * 128 + k] = acc[q];
            }
            __syncthreads();
            if (group == 0 && active) {
                float* out = a.Phi1 + static_cast<size_t>(cur.i) * tp.Q * a.K + k;
#pragma unroll
                for (int q = 0; q < tp.Q; ++q) __stcs(out + static_cast<size_t>(q) * a.K, acc[q] + xchg[q * 128 + k]);
            }
#pragma unroll
            for (int q = 0; q < tp.Q; ++q) acc[q] = 0.f;
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();      // everyone is done with buffer `buf` (accumulator columns, B tile, edge data) before it is staged again
        cur = nxt;
        buf ^= 1;
    }
    __syncthreads();
    if (tid == 0) {
        if (!tiles_ready) mbar_wait(&a_bar, 0);      // a CTA without work still waits for its weight-tile copies before it exits
        if (failed) atomicMax(a.status, failed);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(kCols) : "memory");
}

// =============================================================================================
// Reverse of the tensor product with the radial functions AND their derivatives from the network on the tensor cores.
// Same organisation as tp_forward_rnet_kernel; a batch is 8 edges, and operand B holds for each edge both its hidden
// activations x and their derivatives dx/dr, ordered so that the 16 accumulator columns of a path are, per group g of
// warps, {R(e_2g), R(e_2g+1), R'(e_2g), R'(e_2g+1)}: one 4-column tcgen05.ld per path gives a thread the radial values
// and derivatives of its group's two edges. The adjoint messages go to the senders with red.global.add (float32 path),
// the adjoints of the harmonics and of the edge length are summed over channels as in tp_reverse_kernel.
// =============================================================================================
constexpr int kRnRevEdges = 8;

struct RnEdgeRev {
    float Y[kNumLm];
    float dY[3][kNumLm];
    float ux, uy, uz;
    int j;
};

template <int LF>
struct RnRevSmem {
    static constexpr TPTable tp = make_tp_table(LF);
    static constexpr int kTiles = tp.P * kRnTileBytes;
    static constexpr int kB = 2 * kRnBTileBytes;
    static constexpr int kEdge = 2 * kRnRevEdges * static_cast<int>(sizeof(RnEdgeRev));
    static constexpr int kRed = kRnRevEdges * 4 * 17 * 4;                    // [edge][quadrant][17] partial sums over channels
    static constexpr int kTotal = 1024 + kTiles + kB + kEdge + kRed;
    static constexpr int kDCols = tp.P * kRnEdges;
};

template <int LF>
__global__ void __launch_bounds__(kRnThreads, 1) tp_reverse_rnet_kernel(const TPArgs<float> a, const unsigned char* __restrict__ tiles_image,
                                                                        const RnHidden hd) {
    using S = RnRevSmem<LF>;
    using T = float;
    constexpr TPTable tp = make_tp_table(LF);
    constexpr int kDCols = S::kDCols, kCols = rn_tmem_cols(kDCols);
    extern __shared__ unsigned char rn_smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(rn_smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char* sA = base;
    unsigned char* sB = sA + S::kTiles;
    RnEdgeRev* st = reinterpret_cast<RnEdgeRev*>(sB + S::kB);
    float (*red)[4][17] = reinterpret_cast<float (*)[4][17]>(reinterpret_cast<unsigned char*>(st) + S::kEdge);
    __shared__ __align__(8) unsigned long long a_bar, mma_bar[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int group = warp >> 2, quad = warp & 3, k = quad * 32 + lane;
    const bool active = k < a.K;
    if (tid == 0) {
        failed = 0;
        mbar_init(&a_bar, 1); mbar_init(&mma_bar[0], 1); mbar_init(&mma_bar[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(kCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_slot;
    const uint32_t my_taddr = tmem_d + (static_cast<uint32_t>(quad * 32) << 16) + 4 * group;
    if (tid == 0) {
        mbar_expect_tx(&a_bar, S::kTiles);
        for (int p = 0; p < tp.P; ++p) bulk_copy_g2s(sA + p * kRnTileBytes, tiles_image + static_cast<size_t>(p) * kRnTileBytes, kRnTileBytes, &a_bar);
    }
    bool tiles_ready = false;
    const uint32_t idesc = rn_instr_desc();
    unsigned mma_par[2] = {0u, 0u};

    struct Cursor { int slot; int i; int type_i; long long e0, e_end; };
    auto load_receiver = [&](Cursor& c) {
        if (c.slot < a.N) {
            c.i = a.order ? a.order[c.slot] : c.slot;
            c.type_i = a.node_types[c.i];
            c.e0 = a.first_neigh[c.i];
            c.e_end = a.first_neigh[c.i + 1];
        }
    };
    auto advance = [&](Cursor& c) {
        c.e0 += kRnRevEdges;
        if (c.e0 >= c.e_end) { c.slot += gridDim.x; load_receiver(c); }
    };
    auto stage_batch = [&](const Cursor& c, int buf) {
        const int nb = static_cast<int>(c.e_end - c.e0 < kRnRevEdges ? c.e_end - c.e0 : kRnRevEdges);
        if (warp == kRnThreads / 32 - 1 && lane < kRnRevEdges) {
            RnEdgeRev& s = st[buf * kRnRevEdges + lane];
            if (lane < nb) {
                const long long e = c.e0 + lane;
                const double rr = a.r[e], inv = 1.0 / rr;
                const double ax = a.xyz[3 * e] * inv, ay = a.xyz[3 * e + 1] * inv, az = a.xyz[3 * e + 2] * inv;
                s.ux = float(ax); s.uy = float(ay); s.uz = float(az);
                real_sh3<float, true>(float(ax), float(ay), float(az), float(inv), s.Y, s.dY);
                s.j = a.neigh_indices[e];
            } else {
                s.j = 0;
            }
        }
        {   // operand B: row 4 g + {0, 1} = x of the group's edges 2 g, 2 g + 1; row 4 g + {2, 3} = dx of the same edges
            const int row = tid >> 5, j0 = (tid & 31) * 2;
            const int e = 2 * (row >> 2) + (row & 1);
            float2 v = make_float2(0.f, 0.f), dv = make_float2(0.f, 0.f);
            if (e < nb) rn_hidden_pair(hd, a, c.type_i, c.e0 + e, j0, true, v, dv);
            if (row & 2) v = dv;
            *reinterpret_cast<__half2*>(sB + buf * kRnBTileBytes + rn_swizzled(row, j0)) = __floats2half2_rn(v.x, v.y);
        }
    };
    auto issue_mma = [&](int buf) {
        const uint32_t b_addr = smem_u32(sB + buf * kRnBTileBytes);
#pragma unroll 1
        for (int p = 0; p < tp.P; ++p) {
            const uint32_t a_addr = smem_u32(sA + p * kRnTileBytes);
#pragma unroll
            for (int ks = 0; ks < kRnHidden / 16; ++ks)
                rn_mma(tmem_d + buf * kDCols + p * kRnEdges, tc5_smem_desc(a_addr + ks * 32), tc5_smem_desc(b_addr + ks * 32), idesc, ks > 0 ? 1u : 0u);
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&mma_bar[buf])) : "memory");
    };

    Cursor cur{static_cast<int>(blockIdx.x), 0, 0, 0, 0};
    load_receiver(cur);
    float d[tp.Q];
    int d_slot = -1;            // receiver whose adjoint is in d
    int buf = 0;
    if (cur.slot < a.N) {
        stage_batch(cur, 0);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            if (!mbar_wait(&a_bar, 0)) { atomicMax(&failed, 5); }
            else { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); issue_mma(0); }
        }
        tiles_ready = true;
    }
    while (cur.slot < a.N) {
        Cursor nxt = cur;
        advance(nxt);
        const bool have_next = nxt.slot < a.N;
        if (have_next) stage_batch(nxt, buf ^ 1);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (have_next && tid == 0 && !failed) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            issue_mma(buf ^ 1);
        }
        if (d_slot != cur.slot) {     // first batch of a receiver: its adjoint (overlaps the tensor-core work)
#pragma unroll
            for (int q = 0; q < tp.Q; ++q)
                d[q] = active ? __ldg(a.dPhi1 + (static_cast<size_t>(cur.i) * tp.Q + q) * a.K + k) : 0.f;
            d_slot = cur.slot;
        }
        if (!*reinterpret_cast<volatile int*>(&failed) && !mbar_wait(&mma_bar[buf], mma_par[buf])) atomicMax(&failed, 6);
        mma_par[buf] ^= 1u;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int nb = static_cast<int>(cur.e_end - cur.e0 < kRnRevEdges ? cur.e_end - cur.e0 : kRnRevEdges);
        if (!*reinterpret_cast<volatile int*>(&failed)) {
            uint32_t Rq[tp.P][4];
#pragma unroll
            for (int p = 0; p < tp.P; ++p) rn_ld4_issue(my_taddr + buf * kDCols + p * kRnEdges, Rq[p]);
            float hq[2][tp.nLM];
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                const int e = 2 * group + t;
                const float* hrow = a.H + static_cast<size_t>(st[buf * kRnRevEdges + (e < nb ? e : 0)].j) * tp.nLM * a.K + k;
#pragma unroll
                for (int lm2 = 0; lm2 < tp.nLM; ++lm2) hq[t][lm2] = (e < nb && active) ? __ldg(hrow + static_cast<size_t>(lm2) * a.K) : 0.f;
            }
            rn_ld_wait<tp.P>(Rq);
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                const int e = 2 * group + t;
                if (e < nb) {       // uniform over the warp
                    const RnEdgeRev& s = st[buf * kRnRevEdges + e];
                    float W[kNumLm], fr;
                    if (!active) {
#pragma unroll
                        for (int lm = 0; lm < kNumLm; ++lm) W[lm] = 0.f;
                        fr = 0.f;
                    }
                    if (active) {
                        float h[tp.nLM], msg[tp.nLM], R[tp.P], Rd[tp.P], Y[kNumLm];
#pragma unroll
                        for (int lm2 = 0; lm2 < tp.nLM; ++lm2) h[lm2] = hq[t][lm2];
#pragma unroll
                        for (int p = 0; p < tp.P; ++p) { R[p] = __uint_as_float(Rq[p][t]); Rd[p] = __uint_as_float(Rq[p][2 + t]); }
#pragma unroll
                        for (int lm = 0; lm < kNumLm; ++lm) Y[lm] = s.Y[lm];
                        using ::fma;
                        if constexpr (LF == 0) {
#include "generated/tp_L0_reverse.inc"
                        } else if constexpr (LF == 1) {
#include "generated/tp_L1_reverse.inc"
                        } else {
#include "generated/tp_L2_reverse.inc"
                        }
                        float* arow = a.H_adj + static_cast<size_t>(s.j) * tp.nLM * a.K + k;
#pragma unroll
                        for (int lm2 = 0; lm2 < tp.nLM; ++lm2) atomicAdd(arow + static_cast<size_t>(lm2) * a.K, msg[lm2]);
                    }
                    int idx;
                    const float wsum = warp_reduce_scatter16(W, lane, idx);
                    fr = warp_sum(fr);
                    if ((lane & 1) == 0) red[e][quad][idx] = wsum;
                    if (lane == 0) red[e][quad][16] = fr;
                }
            }
        }
        __syncthreads();
        if (tid < nb && !*reinterpret_cast<volatile int*>(&failed)) {
            // partial force of edge `tid`: nf -= xhat * dE/dr + sum_lm dE/dY_lm grad Y_lm
            const RnEdgeRev& s = st[buf * kRnRevEdges + tid];
            double tr = 0, fx = 0, fy = 0, fz = 0;
            for (int w = 0; w < 4; ++w) tr += red[tid][w][16];
#pragma unroll
            for (int lm = 0; lm < kNumLm; ++lm) {
                double wv = 0;
                for (int w = 0; w < 4; ++w) wv += red[tid][w][lm];
                fx += wv * double(s.dY[0][lm]); fy += wv * double(s.dY[1][lm]); fz += wv * double(s.dY[2][lm]);
            }
            double* nf = a.node_forces + 3 * (cur.e0 + tid);
            nf[0] -= double(s.ux) * tr + fx;
            nf[1] -= double(s.uy) * tr + fy;
            nf[2] -= double(s.uz) * tr + fz;
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        cur = nxt;
        buf ^= 1;
    }
    __syncthreads();
    if (tid == 0) {
        if (!tiles_ready) mbar_wait(&a_bar, 0);
        if (failed) atomicMax(a.status, failed);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(kCols) : "memory");
}

}  // namespace smx
