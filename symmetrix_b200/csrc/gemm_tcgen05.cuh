// float32 channel-mixing GEMMs on the 5th-generation tensor cores (tcgen05.mma, accumulator in tensor memory).
//
// Same problem list as gemm_rows_kernel (rows gathered through (node, sub-row) strides and the type-sorted
// permutation). One CTA of 128 threads owns a 128 x 128 output tile whose accumulator lives in 128 columns of
// TMEM. The k dimension is walked in chunks of 32 floats (one 128-byte swizzle atom per row); for every chunk all
// threads load the A rows and the B columns with ordinary loads, split each float into a TF32 head and a TF32
// remainder (x = hi + lo), and store four operand tiles (A_hi, A_lo, B_hi, B_lo) into shared memory in the
// K-major, 128-byte-swizzled layout the tensor core reads. One thread then issues three MMAs per 8-wide k step
// (lo*hi + hi*lo + hi*hi), which keeps float32-level accuracy, and commits them to an mbarrier. Two shared-memory
// stages are used, so the loads of chunk i+1 overlap the MMAs of chunk i; a stage is rewritten only after the
// commit of its previous use has arrived. Every wait is bounded: if an mbarrier does not flip within the spin
// budget the CTA records an error code, skips further tensor-core work, frees its TMEM and returns.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "kernels.cuh"

namespace smx {

constexpr int kTc5BM = 128, kTc5BN = 128, kTc5BK = 32, kTc5Threads = 128, kTc5Stages = 2;
constexpr int kTc5TileBytes = kTc5BM * kTc5BK * 4;                       // 16 KB per operand tile
constexpr int kTc5StageBytes = 4 * kTc5TileBytes;                        // A_hi, A_lo, B_hi, B_lo
constexpr int kTc5SmemBytes = kTc5Stages * kTc5StageBytes + 1024;        // + slack for 1024-byte alignment
constexpr unsigned kTc5SpinLimit = 1u << 24;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// byte offset of float (row, col) in a K-major tile of 32 floats per row with the 128-byte swizzle:
// rows in groups of 8 (1024 bytes), 16-byte chunk index XOR-ed with the row index inside the group
__device__ __forceinline__ int tc5_swizzled_offset(int row, int col) {
    const int r8 = row & 7;
    const int chunk = (col >> 2) ^ r8;
    return (row >> 3) * 1024 + r8 * 128 + chunk * 16 + (col & 3) * 4;
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

__device__ __forceinline__ bool tc5_wait(uint32_t mbar, uint32_t parity) {
    for (unsigned spin = 0; spin < kTc5SpinLimit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t"
            "}\n"
            : "=r"(done)
            : "r"(mbar), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

// `status` receives a non-zero code if a bounded wait ran out (1: stage reuse, 2: final drain).
__global__ void __launch_bounds__(kTc5Threads) gemm_rows_tcgen05_kernel(const GemmProblem<float>* __restrict__ problems, int* __restrict__ status) {
    const GemmProblem<float> pb = problems[blockIdx.z];
    int node_begin = 0, node_count = pb.num_nodes;
    if (pb.seg) { node_begin = pb.seg[pb.seg_index]; node_count = pb.seg[pb.seg_index + 1] - node_begin; }
    const long long M = static_cast<long long>(node_count) * pb.sub_count;
    const long long row0 = static_cast<long long>(blockIdx.x) * kTc5BM;
    const int col0 = blockIdx.y * kTc5BN;
    if (row0 >= M || col0 >= pb.Nc) return;

    extern __shared__ unsigned char tc5_smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc5_smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    __shared__ __align__(8) unsigned long long mbar[kTc5Stages];
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
        for (int s = 0; s < kTc5Stages; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&mbar[s])) : "memory");
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

    const int num_chunks = (pb.Kd + kTc5BK - 1) / kTc5BK;
    uint32_t phase[kTc5Stages] = {0, 0};
    int uses[kTc5Stages] = {0, 0};
    for (int ch = 0; ch < num_chunks; ++ch) {
        const int stage = ch % kTc5Stages;
        unsigned char* sA_hi = tiles + stage * kTc5StageBytes;
        unsigned char* sA_lo = sA_hi + kTc5TileBytes;
        unsigned char* sB_hi = sA_lo + kTc5TileBytes;
        unsigned char* sB_lo = sB_hi + kTc5TileBytes;
        // the MMAs that read this stage two chunks ago must have completed before it is overwritten
        if (uses[stage] > 0 && !failed) {
            if (!tc5_wait(smem_u32(&mbar[stage]), phase[stage])) { failed = 1; }
            phase[stage] ^= 1;
        }
        __syncthreads();
        const int k0 = ch * kTc5BK;
        // A tile: 128 rows x 32 k, coalesced along k
#pragma unroll 4
        for (int it = 0; it < (kTc5BM * kTc5BK) / kTc5Threads; ++it) {
            const int lin = tid + it * kTc5Threads;
            const int rr = lin >> 5, kk = lin & 31;
            float v = 0.f;
            if (a_base[rr] >= 0 && k0 + kk < pb.Kd) v = pb.A[a_base[rr] + k0 + kk];
            const float hi = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
            const int off = tc5_swizzled_offset(rr, kk);
            *reinterpret_cast<float*>(sA_hi + off) = hi;
            *reinterpret_cast<float*>(sA_lo + off) = v - hi;
        }
        // B tile as [n][k] (K-major): 128 n x 32 k
#pragma unroll 4
        for (int it = 0; it < (kTc5BN * kTc5BK) / kTc5Threads; ++it) {
            const int lin = tid + it * kTc5Threads;
            int nn, kk;
            float v = 0.f;
            if (!pb.transB) {          // B is [Kd][Nc]: read coalesced along n
                kk = lin >> 7; nn = lin & 127;
                if (k0 + kk < pb.Kd && col0 + nn < pb.Nc) v = pb.B[static_cast<size_t>(k0 + kk) * pb.ldb + col0 + nn];
            } else {                   // B is [Nc][Kd]: read coalesced along k
                nn = lin >> 5; kk = lin & 31;
                if (k0 + kk < pb.Kd && col0 + nn < pb.Nc) v = pb.B[static_cast<size_t>(col0 + nn) * pb.ldb + k0 + kk];
            }
            const float hi = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
            const int off = tc5_swizzled_offset(nn, kk);
            *reinterpret_cast<float*>(sB_hi + off) = hi;
            *reinterpret_cast<float*>(sB_lo + off) = v - hi;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic-proxy stores -> visible to the tensor core
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0 && !failed) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_hi = smem_u32(sA_hi), a_lo = smem_u32(sA_lo), b_hi = smem_u32(sB_hi), b_lo = smem_u32(sB_lo);
#pragma unroll
            for (int ks = 0; ks < kTc5BK / 8; ++ks) {
                const uint32_t adv = ks * 32;        // 8 TF32 values = 32 bytes inside the swizzle atom
                const uint32_t first = (ch == 0 && ks == 0) ? 0u : 1u;
                tc5_mma(tmem_d, tc5_smem_desc(a_lo + adv), tc5_smem_desc(b_hi + adv), idesc, first);
                tc5_mma(tmem_d, tc5_smem_desc(a_hi + adv), tc5_smem_desc(b_lo + adv), idesc, 1u);
                tc5_mma(tmem_d, tc5_smem_desc(a_hi + adv), tc5_smem_desc(b_hi + adv), idesc, 1u);
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&mbar[stage])) : "memory");
        }
        uses[stage] += 1;
    }
    // drain: the last commit of every stage that was used
    for (int s = 0; s < kTc5Stages; ++s) {
        if (uses[s] > 0 && !failed) {
            if (!tc5_wait(smem_u32(&mbar[s]), phase[s])) failed = 2;
        }
    }
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (!failed) {
        const long long cb = c_base[warp * 32 + lane];
#pragma unroll
        for (int cc = 0; cc < kTc5BN / 32; ++cc) {
            uint32_t v[32];
            const uint32_t taddr = tmem_d + (static_cast<uint32_t>(warp * 32) << 16) + cc * 32;
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
            if (cb >= 0) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int col = col0 + cc * 32 + j;
                    if (col < pb.Nc) {
                        float* dst = pb.C + cb + col;
                        const float val = __uint_as_float(v[j]);
                        *dst = pb.accumulate ? (*dst + val) : val;
                    }
                }
            }
        }
    } else if (tid == 0) {
        atomicMax(status, failed);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(kTc5BN) : "memory");
}

}  // namespace smx
