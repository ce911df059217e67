// Two rates that bound the tensor-core convolution kernel on one SM, measured with nothing else in the way:
//
//   mma    clocks per 128 x 128 x 16 fp16 MMA unit (tcgen05.mma kind::f16, cta_group::1, both operands in shared
//          memory, K-major without swizzle — the layout of csrc/conv_tc.cu) for the issue patterns of the kernel:
//            n128      27 MMAs of N = 128 per channel block, one thread issuing them back to back
//            conv128   the kernel's pattern for 128 output channels: per filter tap one MMA of N = 256 (hi rows of the
//                      patch against the hi and lo rows of the filter) and one of N = 128 (lo rows against hi rows)
//            conv64    the same for 64 output channels (N = 128 and N = 64)
//            loop128   conv128 issued the way the kernel issues it: a warp-uniform loop, the MMAs under elect.sync,
//                      descriptors formed from run-time arguments, one commit per channel block
//          alone, and beside warps that keep 4-byte cp.async copies into shared memory in flight (the ring loader);
//   copy   bytes per clock one SM gets from cp.async.bulk global -> shared out of an L2-resident buffer the size of a
//          512 -> 512 3x3 filter in fp16 parts, every SM streaming at once, by chunk size and copies in flight.
//
// Every wait is bounded; a wait that runs out sets the status word and the program exits non-zero.
//   nvcc -O3 -std=c++17 -gencode arch=compute_100a,code=sm_100a tc_rates.cu -o tc_rates   (build.py: build_rates_tool)
#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>

namespace {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {      // bounded: about 0.2 s
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try(bar, parity)) return true;
        if (clock64() - t0 > 400000000ll) return false;
    }
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// shared-memory matrix descriptor, K-major, no swizzle: lbo = bytes between the two 16-byte K chunks of a row, sbo = bytes between 8-row groups
__device__ __forceinline__ uint64_t make_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | (uint64_t)((lbo >> 4) & 0x3FFF) << 16 | (uint64_t)((sbo >> 4) & 0x3FFF) << 32 | 1ull << 46;
}
__device__ __forceinline__ uint32_t idesc_of(int n) { return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24); }   // D fp32, A and B fp16, M = 128
__device__ __forceinline__ void mma(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

struct Geometry { int P, Wp; };                 // patch rows staged, width of a padded image row
constexpr int P_MAX = 512;
constexpr int A_BYTES = 2 * P_MAX * 16;         // one part (hi or lo) of the patch: two 16-byte K chunks per row
constexpr int B_TAP = 2 * 256 * 16;             // one filter tap: two K chunks x (128 hi + 128 lo) rows
constexpr int B_BYTES = 9 * B_TAP;              // 73,728 bytes: one channel block of a 3x3 filter for 128 output channels
constexpr int SMEM = 1024 + 2 * A_BYTES + 2 * B_BYTES;
enum { N128 = 0, CONV128 = 1, CONV64 = 2, LOOP128 = 3 };

// the kernel's MMAs of one channel block: descriptors from run-time geometry, as csrc/conv_tc.cu forms them
__device__ __forceinline__ void issue_block(const Geometry& g, uint32_t d, uint32_t a_base, uint32_t b_base, bool first) {
    const uint32_t a_lbo = (uint32_t)g.P * 16u, b_lbo = 256u * 16u;
    const uint64_t a_hi0 = make_desc(a_base, a_lbo, 128), a_lo0 = make_desc(a_base + (uint32_t)g.P * 32u, a_lbo, 128), b0 = make_desc(b_base, b_lbo, 128);
#pragma unroll
    for (int tap = 0; tap < 9; ++tap) {
        const uint32_t a_off = (uint32_t)((tap / 3) * g.Wp + tap % 3);
        const uint64_t b = b0 + (uint64_t)(tap * (B_TAP / 16));
        mma(d, a_hi0 + a_off, b, idesc_of(256), (first && tap == 0) ? 0u : 1u);
        mma(d + 128, a_lo0 + a_off, b, idesc_of(128), 1u);
    }
}

template <int pattern>
__global__ void __launch_bounds__(512) mma_kernel(int blocks, int copiers, const float* src, const Geometry g, long long* clocks, int* status) {
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* done_bar = reinterpret_cast<uint64_t*>(smem);
    uint64_t* block_bar = done_bar + 1;                          // the per-block commits of LOOP128 land here; nobody waits on it
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 64);
    volatile int* finished = reinterpret_cast<volatile int*>(smem + 128);
    unsigned char* A = smem + 1024;
    unsigned char* B0 = A + 2 * A_BYTES;
    unsigned char* B1 = B0 + B_BYTES;                            // the copiers' target
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = tid; i < (2 * A_BYTES + 2 * B_BYTES) / 16; i += blockDim.x) reinterpret_cast<float4*>(A)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (tid == 0) { mbar_init(done_bar, 1); mbar_init(block_bar, 1000000); *finished = 0; asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    if (warp == 0) {
        const long long t0 = clock64();
        if constexpr (pattern == LOOP128) {
            for (int kb = 0; kb < blocks; ++kb) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (elect_one()) {
                    issue_block(g, tmem, smem_u32(A), smem_u32(B0), kb == 0);
                    mma_commit(block_bar);
                }
                __syncwarp();
            }
        } else if (lane == 0) {
            const uint64_t a_hi = make_desc(smem_u32(A), P_MAX * 16, 128), a_lo = make_desc(smem_u32(A + A_BYTES), P_MAX * 16, 128);
            const uint64_t b128 = make_desc(smem_u32(B0), 256 * 16, 128), b64 = make_desc(smem_u32(B0), 128 * 16, 128);
            for (int kb = 0; kb < blocks; ++kb) {
                if constexpr (pattern == N128) {
#pragma unroll
                    for (int i = 0; i < 27; ++i) mma(tmem, a_hi + (uint64_t)((i / 9) * 16 + i % 3), b128 + (uint64_t)((i % 9) * (B_TAP / 16)), idesc_of(128), 1u);
                } else {
#pragma unroll
                    for (int tap = 0; tap < 9; ++tap) {
                        const uint64_t off = (uint64_t)((tap / 3) * 16 + tap % 3);
                        if constexpr (pattern == CONV128) {
                            mma(tmem, a_hi + off, b128 + (uint64_t)(tap * (B_TAP / 16)), idesc_of(256), 1u);
                            mma(tmem + 128, a_lo + off, b128 + (uint64_t)(tap * (B_TAP / 16)), idesc_of(128), 1u);
                        } else {
                            mma(tmem, a_hi + off, b64 + (uint64_t)(tap * (B_TAP / 32)), idesc_of(128), 1u);
                            mma(tmem + 64, a_lo + off, b64 + (uint64_t)(tap * (B_TAP / 32)), idesc_of(64), 1u);
                        }
                    }
                }
            }
        }
        if (lane == 0) {
            mma_commit(done_bar);
            if (!mbar_wait(done_bar, 0)) atomicExch(status, 1);
            clocks[blockIdx.x] = clock64() - t0;
            *finished = 1;
        }
        __syncwarp();
    } else if (warp >= 4 && warp < 4 + copiers) {
        // 4-byte cp.async copies into shared memory, eight per thread in flight, until the issuer is done (bounded)
        const long long t0 = clock64();
        unsigned int turn = tid;
        while (!*finished && clock64() - t0 < 400000000ll) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(reinterpret_cast<float*>(B1) + (tid - 128) + i * 384)),
                             "l"(src + (tid - 128) + i * 384 + (turn & 255) * 4096) : "memory");
            asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
            turn += 7;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
}

// one thread per SM streams `copies` chunks of `chunk` bytes out of src (L2-resident), `depth` of them in flight
__global__ void __launch_bounds__(32) copy_kernel(const float* src, size_t src_bytes, int chunk, int depth, int copies, long long* clocks, int* status) {
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem);           // [depth]
    unsigned char* dst = smem + 1024;
    if (threadIdx.x == 0) {
        for (int d = 0; d < depth; ++d) mbar_init(&bar[d], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const size_t nchunks = src_bytes / chunk;
        size_t at = ((size_t)blockIdx.x * 37) % nchunks;
        bool ok = true;
        const long long t0 = clock64();
        for (int i = 0; i < copies + depth && ok; ++i) {
            const int d = i % depth;
            if (i >= depth) ok = mbar_wait(&bar[d], (uint32_t)(((i / depth) - 1) & 1));
            if (ok && i < copies) {
                bulk_g2s(dst + (size_t)d * chunk, reinterpret_cast<const unsigned char*>(src) + at * chunk, (uint32_t)chunk, &bar[d]);
                if (++at == nchunks) at = 0;
            }
        }
        if (!ok) atomicExch(status, 2);
        clocks[blockIdx.x] = clock64() - t0;
    }
}

}  // namespace

int main() {
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
    if (sms <= 0 || sms > 1024) { printf("no device\n"); return 1; }
    using MmaKernel = void (*)(int, int, const float*, const Geometry, long long*, int*);
    const MmaKernel mma_kernels[4] = {mma_kernel<N128>, mma_kernel<CONV128>, mma_kernel<CONV64>, mma_kernel<LOOP128>};
    for (MmaKernel k : mma_kernels) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    cudaFuncSetAttribute(copy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 1024 + 147456);
    const size_t src_bytes = 9437184;           // 512 x 512 x 9 filter values in two fp16 parts
    float* src; long long* clocks; int* status;
    cudaMalloc(&src, src_bytes); cudaMemset(src, 0, src_bytes);
    cudaMalloc(&clocks, 1024 * sizeof(long long)); cudaMalloc(&status, sizeof(int)); cudaMemset(status, 0, sizeof(int));
    static long long h[1024];
    auto worst = [&](int n) { cudaMemcpy(h, clocks, n * sizeof(long long), cudaMemcpyDeviceToHost); long long m = 0; for (int i = 0; i < n; ++i) m = h[i] > m ? h[i] : m; return m; };
    auto fine = [&]() { int st = 0; cudaError_t e = cudaDeviceSynchronize(); cudaMemcpy(&st, status, sizeof(int), cudaMemcpyDeviceToHost);
                        if (e != cudaSuccess || st) { printf("failed: %s, status %d\n", cudaGetErrorString(e), st); return false; } return true; };

    const char* names[4] = {"n128", "conv128", "conv64", "loop128"};
    const double units[4] = {27, 27, 13.5, 27};                 // 128 x 128 x 16 units per channel block
    const int blocks = 400;
    const Geometry geo[3] = {{512, 16}, {160, 15}, {248, 57}};
    for (int copiers : {0, 12})
        for (int p = 0; p < 4; ++p)
            for (int gi = 0; gi < (p == LOOP128 ? 3 : 1); ++gi) {
                for (int rep = 0; rep < 2; ++rep) mma_kernels[p]<<<sms, 128 + 32 * copiers, SMEM>>>(blocks, copiers, src, geo[gi], clocks, status);
                if (!fine()) return 1;
                printf("mma  %-8s patch rows %3d, image row %2d, %2d cp.async warps beside it: %.1f clocks per 128x128x16 unit (slowest of %d SMs)\n",
                       names[p], geo[gi].P, geo[gi].Wp, copiers, worst(sms) / (blocks * units[p]), sms);
            }
    for (int chunk : {8192, 24576, 73728})
        for (int depth : {1, 2}) {
            const int copies = 600;
            for (int rep = 0; rep < 2; ++rep) copy_kernel<<<sms, 32, 1024 + 147456>>>(src, src_bytes, chunk, depth, copies, clocks, status);
            if (!fine()) return 1;
            const long long m = worst(sms);
            printf("copy chunk %5d bytes, %d in flight: %.1f bytes per clock and SM, %.0f clocks per chunk (slowest of %d SMs, all streaming)\n",
                   chunk, depth, (double)chunk * copies / m, (double)m / copies, sms);
        }
    return 0;
}
