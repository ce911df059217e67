// Tensor-core variant of the core convolution: an implicit GEMM on tcgen05 (sm_100a).
//
// The reference computes this step with fp32 FMAs (its CUDA kernel,
// A100-evaluation/TDC-LAYERS-ORACLE/template_benchmark_cudnn.template:365-402) or leaves it
// to cuDNN (inference/TKConv.py:92-93); it has no tensor-core path.  On B200 the fp32 FMA
// pipe is held back by the shared-memory return path, while the 5th-generation tensor cores
// are idle, so this file maps the same convolution onto tcgen05.mma kind::tf32:
//
//   D[128 positions][NT channels] += A_tap[128 positions][8 channels] * B_tap[8 channels][NT]
//
// summed over the R*S taps and all channel blocks, accumulator in tensor memory.
//
//   * Positions.  Each image is laid out (conceptually) row by row with ONE zero column
//     after every row and one zero row after the image (row pitch Wp = W + 1).  In that
//     layout the input of output position g for tap (r, s) is position
//     g + (r-1)*Wp + (s-1), for every g — the halo of a row is the zero column of its
//     neighbour.  A CTA owns 128 consecutive positions (possibly spanning images), stages
//     the patch of positions it needs once per channel block, and every tap reads the same
//     patch at a different row offset.  Outputs that fall on a zero column/row are dropped.
//   * Shared-memory operand layout: K-major, no swizzle, [channel/4][row][4 floats]: a
//     core matrix (8 rows x 16 bytes) is contiguous for ANY starting row, which is what lets
//     the nine taps address one patch with descriptors that differ only in their start.
//   * Precision.  mode 3 ("3xTF32"): every operand is split x = hi + lo with hi = tf32(x),
//     and hi*hi + hi*lo + lo*hi is accumulated in fp32 — products are then exact to ~2^-21,
//     i.e. fp32-level results (tests hold it to the fp32 bar of 1e-5).  mode 1: plain TF32,
//     one MMA per tap and step, reported separately at 5e-3.
//   * The filter is pre-arranged once (tdc_tc_prepare_weights) into the exact shared-memory
//     image of each (channel block, output block), so staging it is one plain bulk copy
//     (cp.async.bulk into this CTA's shared memory) that completes on an mbarrier.
//   * Every wait on an mbarrier is bounded; a wait that runs out records a status word,
//     the CTA skips to its clean-up (tensor memory is freed) and returns.
#include <cuda.h>            // CUtensorMap and its enums (types only: the encoder is looked up at run time)
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>
#include <utility>
#include "../../include/tdc_b200.h"

namespace tdc_tc {

constexpr int M_TILE   = 128;   // positions per CTA = MMA M
constexpr int CB       = 8;     // 4-byte words per operand row and K step (32 bytes): 8 TF32 channels, or 16 fp16 channels
constexpr int BOXW     = 32;    // pixels per row of a bulk-tensor box (128 bytes)
constexpr int BOXC     = 16;    // channels per box = one fp16 K step
// channels of one K step: kind::tf32 contracts 8 per MMA, kind::f16 16 (the operand bytes are the same)
template <bool F16> struct KStep { static constexpr int CH = F16 ? 16 : 8; };
constexpr int LOADERS  = 256;   // threads of warps 0-7, which stage the input patch
constexpr int THREADS  = 384;   // + warps 8-11: MMA issuers (lane 0 of each), everyone drains tensor memory

// Division of a non-negative number below 2^31 by a fixed divisor as one widening multiply and a shift: the index
// arithmetic of the loaders, the producer and the epilogue divides by the row pitch, the positions per image and the
// number of output-channel blocks once or more per tile and work item, and an integer division is 20 (32-bit) to
// 100 (64-bit) dependent instructions of a single warp.  mul = floor(2^(31+s) / d) + 1 with 2^(s-1) < d <= 2^s:
// n * mul >> (31 + s) == n / d for every 0 <= n < 2^31 (the excess mul * d - 2^(31+s) is at most d <= 2^s, so the
// product overshoots n / d by less than 1 / d).
struct FastDiv { uint32_t mul, shift; };
inline FastDiv fastdiv_make(uint32_t d) {
    uint32_t s = 0;
    while ((1ull << s) < d) ++s;
    FastDiv f;
    f.mul = (uint32_t)(((1ull << (31 + s)) / d) + 1ull);
    f.shift = 31 + s;
    return f;
}
__host__ __device__ __forceinline__ uint32_t fastdiv(uint32_t n, FastDiv f) { return (uint32_t)(((unsigned long long)n * f.mul) >> f.shift); }

struct Args {
    const float* x;        // [B][C][H][W]
    const float* wt;       // pre-arranged filter, see prepare kernel
    float*       y;        // [B][K][H][W]
    const float* scale; const float* bias; const float* residual;
    int relu;
    int epi_vec;           // scale and bias are 16-byte aligned (or absent): whole chunks read them as 16-byte words
    int B, C, H, W, K;     // H, W: the OUTPUT image (equal to the input image unless a 1x1 filter is strided)
    int stride, Win;       // input step per output position and input row length
    long long HWin;        // input image size (channel pitch of x)
    int gather, gR, gS, gpad, Hin;   // general plan: the channels the MMAs see are (input channel, filter row, filter column) triples
    int gpadx, gpair;      // column padding as the loaders see it (strided rows: less the plan's phase); stride 2: both phases by one 8-byte copy
    int taps_r;            // R (= S): 1 or 3
    int halo, shift;       // patch rows beyond a tile's positions, and how far ahead of the tile the patch starts
    float rz_unit;         // expected truncation loss of a sum per channel block (see load_chunk); 0: none put back
    int Wp, Lp;            // row pitch and positions per image of the padded position space
    int Hp;                // Lp / Wp: rows of a padded image
    FastDiv fd_Wp, fd_Lp, fd_nocb;   // the divisors of the index arithmetic (valid while positions and tiles stay below 2^31: `small`)
    int small;             // total_pos and ntiles fit 31 bits: the kernels divide by multiplication
    int P;                 // patch rows staged per CTA (multiple of 8)
    int nkb;               // channel blocks
    int n_ocb;             // output-channel blocks
    int hl;                // 2: hi/lo split (3xTF32, 3xFP16), 1: plain TF32
    int ns;                // stages
    int nmain;             // 1 or 2 main accumulators per position tile (2: channel blocks alternate)
    int tile_cols;         // tensor-memory columns per position tile: 2*NT, or 4*NT with two mains
    int tmem_cols;         // allocation (power of two >= 32)
    long long total_pos;   // B * Lp
    int nbuf;              // persistent kernel: accumulator buffers in tensor memory (1 or 2)
    int depth;             // persistent kernel: slots of the raw-input ring (cp.async groups in flight)
    int kps;               // persistent kernel: channel blocks per shared-memory stage
    long long full_groups, tail_first_pt, pt_total;   // persistent kernel: tile list (see tile_of)
    int tail_cnt;
    long long ntiles;      // persistent kernel: position tiles x output-channel blocks
    int nseg, seg_blocks;  // persistent kernel: the channel blocks of a tile are accumulated in nseg runs of seg_blocks
                           // blocks; each run starts fresh accumulators and is added to y in fp32 by the epilogue
    int nbox_cap;          // bulk-tensor loader: boxes a raw slot holds
    int step_y, step_x;    // bulk-tensor loader: 256 positions = step_y padded rows + step_x columns
    // fp16 operands: the input is scaled by a power of two into fp16's range (which ends at 65504), the filter likewise
    // when it is prepared, and the epilogue undoes both.  fp16 keeps its 11 significant bits over 30 binades, so the
    // scale need not be exact: given a bound of |x| it goes just under 2^14; without one, every CTA takes the largest
    // of 1500 - 2000 elements spread over x (four per thread of its draining warps) and puts that at 2^8, which leaves a factor of 256 for values the sample
    // missed.  An input beyond even that turns into infinities, which the epilogue sees in its outputs and reports
    // through the status word (2): never a silent wrong result.
    const float* x_absmax; // [ABSMAX_SLOTS] partial maxima of |x| (every entry valid; the largest one counts), or nullptr
    long long x_count;     // elements of x
    const float* w_scale;  // [1] the power of two the prepared filter was multiplied by
    float*       y_absmax; // [ABSMAX_SLOTS] or nullptr: partial maxima of |y| for the next layer (entry = CTA, rest zeroed)
    int* status;           // device status word: 0 ok, else first failure code
};
constexpr int ABSMAX_SLOTS = 1024;


// The power of two that brings a magnitude m just under 2^target; 1 for a zero or non-finite m.
__host__ __device__ __forceinline__ float range_scale(float m, int target = 14) {
    if (!(m > 0.f) || !(m < 3.0e38f)) return 1.f;
    int e;
    frexpf(m, &e);                                  // m = f * 2^e, 0.5 <= f < 1
    int k = target - e;
    k = k < -60 ? -60 : (k > 60 ? 60 : k);
    return ldexpf(1.f, k);
}

// The largest of the ABSMAX_SLOTS partial maxima, by the first 256 threads of a block (all threads must call it).
__device__ __forceinline__ float absmax_of(const float* slots, unsigned int* scratch /* one shared word */) {
    if (threadIdx.x == 0) *scratch = 0;
    __syncthreads();
    if (threadIdx.x < 256) {
        unsigned int m = 0;
#pragma unroll
        for (int i = 0; i < ABSMAX_SLOTS / 256; ++i) m = max(m, __float_as_uint(slots[threadIdx.x + i * 256]) & 0x7fffffffu);
        m = __reduce_max_sync(0xffffffffu, m);
        if ((threadIdx.x & 31) == 0) atomicMax(scratch, m);
    }
    __syncthreads();
    const float m = __uint_as_float(*scratch);
    __syncthreads();                               // every thread has read the word: the caller may reuse it
    return m;
}

// The range of the input of a launch with fp16 operands, found by `threads` threads of the block (whole warps; `idx` =
// the thread's index among them): the largest of the given ABSMAX_SLOTS partial maxima of |x|, or, without such a bound,
// the largest magnitude among RANGE_PER_THREAD elements per thread spread evenly over x (all of x when it is shorter).
// Two steps, so that the loads (one memory round trip, cold pages included) run under whatever the caller does between
// them: range_load issues this thread's loads and hands back the raw words — nothing uses the loaded registers until
// range_max reduces them.
constexpr int RANGE_PER_THREAD = 4;
__device__ __forceinline__ void range_load(const float* slots, const float* x, long long n, int idx, int threads, unsigned int (&raw)[RANGE_PER_THREAD]) {
    if (slots) {
#pragma unroll
        for (int i = 0; i < RANGE_PER_THREAD; ++i) raw[i] = idx + i * threads < ABSMAX_SLOTS ? __float_as_uint(slots[idx + i * threads]) : 0u;
    } else {
        const int want = RANGE_PER_THREAD * threads;
        const long long step = n > want ? n / want : 1;
#pragma unroll
        for (int i = 0; i < RANGE_PER_THREAD; ++i) {
            const long long k = (long long)(idx + i * threads) * step;
            raw[i] = k < n ? __float_as_uint(__ldg(x + k)) : 0u;
        }
    }
}
// `scratch` was zeroed before the block's last barrier.  The threads that loaded reduce into it and meet the threads
// that only need the result (range_wait) at named barrier 1, `meeting` threads in all; the rest of the block does not wait.
__device__ __forceinline__ float range_max(const unsigned int (&raw)[RANGE_PER_THREAD], unsigned int* scratch, int meeting) {
    unsigned int mine = 0;
#pragma unroll
    for (int i = 0; i < RANGE_PER_THREAD; ++i) mine = max(mine, raw[i] & 0x7fffffffu);
    const unsigned int m = __reduce_max_sync(0xffffffffu, mine);
    if ((threadIdx.x & 31) == 0 && m) atomicMax(scratch, m);
    asm volatile("bar.sync 1, %0;" ::"r"(meeting) : "memory");
    return __uint_as_float(*reinterpret_cast<volatile unsigned int*>(scratch));
}
__device__ __forceinline__ float range_wait(unsigned int* scratch, int meeting) {
    asm volatile("bar.sync 1, %0;" ::"r"(meeting) : "memory");
    return __uint_as_float(*reinterpret_cast<volatile unsigned int*>(scratch));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait: true when the phase with `parity` has completed, false after ~1 s.
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    if (mbar_try(bar, parity)) return true;          // the common case costs no clock read
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try(bar, parity)) return true;
        if (clock64() - t0 > 2000000000ll) return false;
    }
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// 4-byte asynchronous copy global -> shared; `real` false writes a zero and reads nothing.
__device__ __forceinline__ void cp_async4(void* dst, const void* src, bool real) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(real ? 4u : 0u) : "memory");
}
// Wait until at most n of this thread's most recent cp.async groups are still in flight (n <= 7).
__device__ __forceinline__ void cp_async_wait_pending(int n) {
    switch (n) {
        case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
        case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
        case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
        case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
        case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
        case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
        case 6: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
        default: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
    }
}
__device__ __forceinline__ float to_tf32(float v) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return __uint_as_float(r);
}

// One patch row of one channel block -> the operand layout of a stage: two 16-byte words (the two core matrices of a
// K step) of the hi part at A + ((q*P + pp) << 2) and, with split operands, of the lo part 8*P words further on.
// TF32: word q holds channels 4q..4q+3 as fp32 bit patterns with 10 mantissa bits; lo = c - hi.
// FP16: word q holds channels 8q..8q+7 as halves; lo = (c - hi) * 2^11, which keeps it in fp16's normal range
// for every c whose hi part is (the epilogue divides the small accumulator by 2^11 again).
template <bool F16>
__device__ __forceinline__ void store_row(float* A, int P, int hl, int pp, const float (&c)[KStep<F16>::CH], float xs = 1.f) {
    if constexpr (F16) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            uint32_t h[4], l[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float c0 = c[8 * q + 2 * k] * xs, c1 = c[8 * q + 2 * k + 1] * xs;     // xs: the range scaling, a power of two
                const __half2 hh = __floats2half2_rn(c0, c1);
                const float2 hf = __half22float2(hh);
                const __half2 ll = __floats2half2_rn((c0 - hf.x) * 2048.f, (c1 - hf.y) * 2048.f);
                h[k] = *reinterpret_cast<const uint32_t*>(&hh);
                l[k] = *reinterpret_cast<const uint32_t*>(&ll);
            }
            *reinterpret_cast<uint4*>(A + ((q * P + pp) << 2)) = make_uint4(h[0], h[1], h[2], h[3]);
            if (hl == 2) *reinterpret_cast<uint4*>(A + CB * P + ((q * P + pp) << 2)) = make_uint4(l[0], l[1], l[2], l[3]);
        }
    } else {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            float4 hi;
            hi.x = to_tf32(c[4 * q]); hi.y = to_tf32(c[4 * q + 1]); hi.z = to_tf32(c[4 * q + 2]); hi.w = to_tf32(c[4 * q + 3]);
            *reinterpret_cast<float4*>(A + ((q * P + pp) << 2)) = hi;
            if (hl == 2)
                *reinterpret_cast<float4*>(A + CB * P + ((q * P + pp) << 2)) =
                    make_float4(c[4 * q] - hi.x, c[4 * q + 1] - hi.y, c[4 * q + 2] - hi.z, c[4 * q + 3] - hi.w);
        }
    }
}

// Shared-memory matrix descriptor: K-major, no swizzle.  lbo = bytes between the two core
// matrices of one K step (channels 0-3 / 4-7), sbo = bytes between 8-row groups.
__device__ __forceinline__ uint64_t make_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
    d |= 1ull << 46;                 // descriptor version of sm_100
    return d;                        // layout type 0 (no swizzle), base offset 0
}
template <bool F16>
__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    if constexpr (F16)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                     ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                     ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 32 consecutive columns of this warp's 32 tensor-memory lanes -> 32 registers per thread.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}

// ... and 16 of them (the persistent kernel's epilogue works in half chunks: it has fewer registers per thread).
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld32(taddr, r); }
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}

// One lane of a converged warp, chosen by the hardware.  The MMA issue loops run warp-uniform
// (every lane waits on the barriers and computes the same descriptors) and only the MMA and
// commit instructions sit under this predicate: operands the compiler can prove warp-uniform
// stay in uniform registers, which is what the tensor-core instructions read.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

// Instruction descriptor: D fp32, A and B tf32 (format 2) or fp16 (format 0), both K-major, M = 128, N = n.
template <bool F16>
__device__ __forceinline__ uint32_t make_idesc(int n) {
    const uint32_t fmt = F16 ? 0u : 2u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(M_TILE >> 4) << 24);
}

// The MMAs of one channel block (stage) of one position tile.  `a_base` / `b_base`: shared
// addresses of the stage's patch and filter; `row16`: first patch row of the tile (the unit
// of a start-address step is 16 bytes = one patch row of one core matrix); `odd`: this block
// is an odd channel block of its run; `first`: it starts the accumulation of the accumulator it feeds.
template <int NT, int TAPS, bool F16 = false>
__device__ __forceinline__ void issue_block(const Args& a, uint32_t d_main, uint32_t a_base, uint32_t b_base, uint32_t row16,
                                            bool odd, bool first) {
    // leading byte offset = distance between the two core matrices of a K step (the two 16-byte halves of an operand
    // row), stride byte offset = distance between groups of 8 rows (verified on a B200 against the fp64 oracle)
    const uint32_t a_lbo = (uint32_t)a.P * 16u, b_lbo = (uint32_t)(a.hl * NT) * 16u, sbo = 128u;
    const uint32_t idesc_n = make_idesc<F16>(NT), idesc_2n = make_idesc<F16>(2 * NT);
    const uint64_t a_hi0 = make_desc(a_base, a_lbo, sbo) + row16;
    const uint64_t a_lo0 = make_desc(a_base + (uint32_t)(CB * a.P) * 4u, a_lbo, sbo) + row16;
    const uint64_t b_hi0 = make_desc(b_base, b_lbo, sbo);       // rows 0..NT-1 hi, NT..2NT-1 lo
    const uint32_t b_tap = (uint32_t)((CB / 4) * a.hl * NT);    // filter rows per tap, in 16-byte units
    if (a.hl == 1) {
#pragma unroll
        for (int tap = 0; tap < TAPS; ++tap) {
            const uint32_t a_off = TAPS == 9 ? (uint32_t)((tap / 3) * a.Wp + tap % 3) : (uint32_t)tap;   // 3x3: rows and columns; else: columns
            mma_tf32<F16>(d_main, a_hi0 + a_off, b_hi0 + tap * b_tap, idesc_n, (first && tap == 0) ? 0u : 1u);
        }
    } else if (a.nmain == 2 && odd) {
        // odd channel block: second main accumulator; the lo rows of the filter start NT rows (NT x 16 bytes) in
#pragma unroll
        for (int tap = 0; tap < TAPS; ++tap) {
            const uint32_t a_off = TAPS == 9 ? (uint32_t)((tap / 3) * a.Wp + tap % 3) : (uint32_t)tap;   // 3x3: rows and columns; else: columns
            const uint64_t b_hi = b_hi0 + tap * b_tap;
            mma_tf32<F16>(d_main + 2 * NT, a_hi0 + a_off, b_hi, idesc_n, (first && tap == 0) ? 0u : 1u);   // main1 += hi*hi
            mma_tf32<F16>(d_main + NT, a_hi0 + a_off, b_hi + (uint64_t)NT, idesc_n, 1u);                   // small += hi*lo
            mma_tf32<F16>(d_main + NT, a_lo0 + a_off, b_hi, idesc_n, 1u);                                  // small += lo*hi
        }
    } else {
#pragma unroll
        for (int tap = 0; tap < TAPS; ++tap) {
            const uint32_t a_off = TAPS == 9 ? (uint32_t)((tap / 3) * a.Wp + tap % 3) : (uint32_t)tap;   // 3x3: rows and columns; else: columns
            const uint64_t b_hi = b_hi0 + tap * b_tap;
            mma_tf32<F16>(d_main, a_hi0 + a_off, b_hi, idesc_2n, (first && tap == 0) ? 0u : 1u);           // main += hi*hi, small += hi*lo
            mma_tf32<F16>(d_main + NT, a_lo0 + a_off, b_hi, idesc_n, 1u);                                  // small += lo*hi
        }
    }
}

// 32 output channels of this thread's position: tensor memory -> registers, with the
// accumulators of the split (main + small, + second main) added in fp32.  `blocks`: channel
// blocks of the run these accumulators hold (the second main exists from two blocks on).
// With fp16 operands the lo halves were scaled by 2^11 on both sides (so that they stay
// clear of fp16's subnormal range); the small accumulator carries that factor.
template <int NT, bool F16 = false, int W = 32>
__device__ __forceinline__ void load_chunk(const Args& a, uint32_t taddr, uint32_t (&r)[W], int blocks, float inv = 1.f) {
    tmem_ld(taddr, r);
    if (a.hl == 2) {
        uint32_t r2[W];
        tmem_ld(taddr + NT, r2);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        // The tensor core truncates its fp32 running sum toward zero at every accumulation, which shrinks a sum of n
        // accumulations by n * 2^-26 on average (measured: -1.55e-8 .. -1.72e-8 per accumulation for 18..288 of
        // them, whatever the layer or the sign pattern of its input).  `rz_unit` = 2^-26 x accumulations per channel
        // block and main accumulator (0 = leave the sums as they are): the expected loss is put back here, so that the
        // error left has no sign and does not add up from layer to layer of a network.
        const float comp = fmaf(a.rz_unit, (float)blocks, 1.f);
        if constexpr (F16) {
            // `inv` undoes the range scaling of input and filter; the small accumulator also carries the 2^11 of the lo halves
            const float inv_small = inv * (1.f / 2048.f);
            inv *= comp;
#pragma unroll
            for (int k = 0; k < W; ++k) r[k] = __float_as_uint(fmaf(__uint_as_float(r2[k]), inv_small, __uint_as_float(r[k]) * inv));
        } else {
            inv = comp;
#pragma unroll
            for (int k = 0; k < W; ++k) r[k] = __float_as_uint(fmaf(__uint_as_float(r[k]), inv, __uint_as_float(r2[k])));
        }
        if (a.nmain == 2 && blocks > 1) {          // second main accumulator (odd channel blocks)
            tmem_ld(taddr + 2 * NT, r2);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int k = 0; k < W; ++k) r[k] = __float_as_uint(fmaf(__uint_as_float(r2[k]), inv, __uint_as_float(r[k])));
        }
    } else {
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    }
}

// ... and registers -> y (NCHW: the lanes of a warp hold consecutive positions, so every
// store instruction writes one contiguous run).  `out_off` < 0: the position is padding.
// Called by whole warps.  With the fused options, lane k fetches scale and bias of channel
// oc0 + k once and the others get them by shuffle, and the 32 residual values are loaded
// before the first store (y and the residual may be the same buffer as far as the compiler
// knows, so loads placed between the stores would each wait out a memory round trip).
// `accum`: these accumulators are a later run of the tile's channel blocks: y already holds the sum of the
// earlier runs (written by this same thread) and is added first.  `final`: this is the tile's last run, the
// fused options apply; otherwise the bare partial sum is stored.
template <int W = 32>
__device__ __forceinline__ void store_chunk(const Args& a, const uint32_t (&r)[W], long long out_off, int oc0, long long HW,
                                            bool accum = false, bool final = true, float* vmax = nullptr) {
    const int lane = threadIdx.x & 31;
    const bool live = out_off >= 0;
    const long long o0 = (live ? out_off : 0) + (long long)oc0 * HW;
    float* yp = a.y + o0;
    const int n = a.K - oc0;                      // channels of this chunk that exist
    if (n >= W && !accum && (!final || (!a.scale && !a.bias && !a.residual && !a.relu))) {
        if (live) {
#pragma unroll
            for (int k = 0; k < W; ++k) { *yp = __uint_as_float(r[k]); yp += HW; }
            if (vmax) {                               // magnitudes compare like their bit patterns
                unsigned int m = __float_as_uint(*vmax);
#pragma unroll
                for (int k = 0; k < W; ++k) m = max(m, r[k] & 0x7fffffffu);
                *vmax = __uint_as_float(m);
            }
        }
        return;
    }
    float v[W];
#pragma unroll
    for (int k = 0; k < W; ++k) v[k] = __uint_as_float(r[k]);
    if (accum && live) {
        const float* q = yp;                       // one stepping pointer, not 32 addresses
#pragma unroll
        for (int k = 0; k < W; ++k) { if (k < n) v[k] += *q; q += HW; }
    }
    if (!final) {
        if (live) {
#pragma unroll
            for (int k = 0; k < W; ++k)
                if (k < n) yp[k * HW] = v[k];
        }
        return;
    }
    if (n >= W && a.epi_vec) {
        // a whole chunk, 16-byte aligned scale / bias: eight warp-uniform 16-byte loads each instead of 32 shuffles
        if (a.scale) {
            const float4* sp = reinterpret_cast<const float4*>(a.scale + oc0);
#pragma unroll
            for (int k4 = 0; k4 < W / 4; ++k4) {
                const float4 t = __ldg(sp + k4);
                v[4 * k4] *= t.x; v[4 * k4 + 1] *= t.y; v[4 * k4 + 2] *= t.z; v[4 * k4 + 3] *= t.w;
            }
        }
        if (a.bias) {
            const float4* bp = reinterpret_cast<const float4*>(a.bias + oc0);
#pragma unroll
            for (int k4 = 0; k4 < W / 4; ++k4) {
                const float4 t = __ldg(bp + k4);
                v[4 * k4] += t.x; v[4 * k4 + 1] += t.y; v[4 * k4 + 2] += t.z; v[4 * k4 + 3] += t.w;
            }
        }
    } else {
        const float sc = (a.scale && lane < n && lane < W) ? __ldg(a.scale + oc0 + lane) : 1.f;
        const float bi = (a.bias && lane < n && lane < W) ? __ldg(a.bias + oc0 + lane) : 0.f;
        if (a.scale) {
#pragma unroll
            for (int k = 0; k < W; ++k) v[k] *= __shfl_sync(0xffffffffu, sc, k);
        }
        if (a.bias) {
#pragma unroll
            for (int k = 0; k < W; ++k) v[k] += __shfl_sync(0xffffffffu, bi, k);
        }
    }
    if (a.residual && live) {
        const float* rp = a.residual + o0;
        float rv[W];
#pragma unroll
        for (int k = 0; k < W; ++k) rv[k] = k < n ? rp[k * HW] : 0.f;
#pragma unroll
        for (int k = 0; k < W; ++k) v[k] += rv[k];
    }
    if (a.relu) {
#pragma unroll
        for (int k = 0; k < W; ++k) v[k] = fmaxf(v[k], 0.f);
    }
    if (vmax && live) {                              // largest stored magnitude (as a bit pattern: a NaN must not get lost)
        unsigned int m = __float_as_uint(*vmax);
#pragma unroll
        for (int k = 0; k < W; ++k) m = max(m, k < n ? (__float_as_uint(v[k]) & 0x7fffffffu) : 0u);
        *vmax = __uint_as_float(m);
    }
    if (live) {
        if (n >= W) {
#pragma unroll
            for (int k = 0; k < W; ++k) { *yp = v[k]; yp += HW; }
        } else {
#pragma unroll
            for (int k = 0; k < W; ++k)
                if (k < n) yp[k * HW] = v[k];
        }
    }
}

// NT output channels and MT tiles of 128 positions per CTA.  Tensor memory holds, per
// position tile, NT "main" columns (hi*hi) followed by NT "small" columns (hi*lo + lo*hi):
// the small products never pass through the large running sum, whose rounding inside the
// tensor core would otherwise swamp them, and fp32 adds main + small once in the epilogue.
// The tensor core rounds its running sum at every accumulation, so for long reductions
// (many channel blocks x taps) the host asks for TWO main accumulators per tile, fed by even
// and odd channel blocks ([main0 | small | main1] in tensor memory): each running sum is half
// as long, and the epilogue adds them in fp32.
//
// Warp roles.  Warps 0-7 (LOADERS) stage the input patch: global -> registers -> hi/lo split
// -> shared, and one of their threads starts the filter's bulk copy; they run up to `ns`
// stages ahead.  Lane 0 of warp 8+mt (ISSUERS) issues the MMAs of position tile mt as soon as
// a stage's mbarrier says the patch is stored and the filter has landed, and commits to the
// mbarrier that hands the stage back.  There is no CTA-wide barrier in the main loop.  All
// twelve warps drain tensor memory in the epilogue.
template <int NT, int MT, int TAPS, bool VEC>
__global__ void __launch_bounds__(THREADS) conv_tc_kernel(const Args a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    // carve: barriers | tmem slot | stages { A[hl][CB/4][P][4], B[tap][CB/4][hl*NT][4] }
    uint64_t* full_bar  = reinterpret_cast<uint64_t*>(smem_raw);           // [ns] patch stored + filter landed
    uint64_t* empty_bar = full_bar + 4;                                     // [ns] MMAs of the stage done
    uint64_t* done_bar  = empty_bar + 4;                                    // all MMAs done
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done_bar + 1);
    int*      abort_flag = reinterpret_cast<int*>(tmem_slot + 1);
    float*    stage0    = reinterpret_cast<float*>(smem_raw + 128);

    constexpr int PPT = 3;      // patch rows per loader thread: the host keeps P <= 3 * LOADERS
    const uint32_t TMEM_COLS = (uint32_t)a.tmem_cols;
    const int a_floats = a.hl * CB * a.P;                  // A part of a stage
    const int b_floats = a.hl * TAPS * CB * NT;            // B part of a stage
    const int stage_floats = a_floats + b_floats;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const int ocb = blockIdx.x % a.n_ocb;
    const long long g0 = (long long)(blockIdx.x / a.n_ocb) * (MT * M_TILE);   // first output position
    const long long gp0 = g0 - a.shift;                                    // position of patch row 0
    const long long HW = (long long)a.H * a.W;

    if (tid == 0) {
        // full: every loader warp arrives once (lane 0, after the warp's stores), plus the arrive that announces the filter's bytes;
        // empty / done: one commit per issuing thread
        for (int s = 0; s < a.ns; ++s) { mbar_init(&full_bar[s], LOADERS / 32 + 1); mbar_init(&empty_bar[s], MT); }
        mbar_init(done_bar, MT);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    const uint32_t b_bytes = (uint32_t)b_floats * 4u;
    const float* wt_cta = a.wt + (long long)ocb * a.nkb * b_floats;

    if (warp < 8) {
        // ================= loaders =================
        // Two channel blocks of input are always in flight in registers (blocks kb and kb+1 are
        // loaded while kb-1 is being split and stored), and the filter copies run `ns` stages ahead.
        // ring positions are counters that wrap, not kb % ns: these loops are bound by instruction latency
        int st_idx = 0, st_use = 0;                     // stage to fill next, parity of its use count
        auto open_stage = [&](int kb) -> float* {       // wait until the stage is free, start its filter copy
            const int s = st_idx;
            float* A = stage0 + (long long)s * stage_floats;
            // use number u of a stage waits for the MMAs of use u-1; the first use passes at once
            if (!mbar_wait(&empty_bar[s], (uint32_t)(st_use ^ 1))) { *abort_flag = 1; return nullptr; }
            if (tid == 0) {
                mbar_expect_tx(&full_bar[s], b_bytes);
                bulk_g2s(A + a_floats, wt_cta + (long long)kb * b_floats, b_bytes, &full_bar[s]);
            }
            return A;
        };
        auto close_stage = [&](int kb) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> visible to the tensor core
            __syncwarp();                                                  // one arrival per warp: 8 instead of 256 updates of one barrier
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&full_bar[st_idx])) : "memory");
            if (++st_idx == a.ns) { st_idx = 0; st_use ^= 1; }
        };
        auto put = [&](float* A, int q, int pp, float c0, float c1, float c2, float c3) {   // 4 channels of one patch row
            float4 hi;
            hi.x = to_tf32(c0); hi.y = to_tf32(c1); hi.z = to_tf32(c2); hi.w = to_tf32(c3);
            *reinterpret_cast<float4*>(A + ((q * a.P + pp) << 2)) = hi;
            if (a.hl == 2)
                *reinterpret_cast<float4*>(A + CB * a.P + ((q * a.P + pp) << 2)) = make_float4(c0 - hi.x, c1 - hi.y, c2 - hi.z, c3 - hi.w);
        };
        if constexpr (VEC) {
            // 1x1 filter, H*W a multiple of 4: a thread owns 4 consecutive positions x 4 channels of
            // the block; four 16-byte loads (one per channel), transposed in registers into four
            // 16-byte stores (one per position)
            constexpr int NI = (MT * M_TILE / 2 + LOADERS - 1) / LOADERS;     // items per thread
            long long off[NI];
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                const int item = tid + i * LOADERS, quad = item >> 1;
                off[i] = -1;
                if (quad * 4 < a.P) {
                    const long long g = g0 + quad * 4;
                    if (g < a.total_pos) { const long long b = g / a.Lp; off[i] = b * a.C * HW + (g - b * a.Lp); }
                }
            }
            float4 va[NI][4], vb[NI][4];
            auto load = [&](int kb, float4 (&v)[NI][4]) {
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    const int c0 = kb * CB + ((tid + i * LOADERS) & 1) * 4;
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        v[i][j] = (off[i] >= 0 && c0 + j < a.C) ? __ldg(reinterpret_cast<const float4*>(a.x + off[i] + (long long)(c0 + j) * HW))
                                                                 : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            };
            auto stage = [&](int kb, float4 (&v)[NI][4]) -> bool {
                float* A = open_stage(kb);
                if (!A) return false;
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    const int item = tid + i * LOADERS, q = item & 1, pp = (item >> 1) * 4;
                    if (pp < a.P) {
                        put(A, q, pp + 0, v[i][0].x, v[i][1].x, v[i][2].x, v[i][3].x);
                        put(A, q, pp + 1, v[i][0].y, v[i][1].y, v[i][2].y, v[i][3].y);
                        put(A, q, pp + 2, v[i][0].z, v[i][1].z, v[i][2].z, v[i][3].z);
                        put(A, q, pp + 3, v[i][0].w, v[i][1].w, v[i][2].w, v[i][3].w);
                    }
                }
                close_stage(kb);
                return true;
            };
            load(0, va);
            if (a.nkb > 1) load(1, vb);
            for (int kb = 0; kb < a.nkb; kb += 2) {
                if (!stage(kb, va)) break;
                if (kb + 2 < a.nkb) load(kb + 2, va);
                if (kb + 1 < a.nkb) {
                    if (!stage(kb + 1, vb)) break;
                    if (kb + 3 < a.nkb) load(kb + 3, vb);
                }
            }
        } else {
            long long src_off[PPT];        // global offset of channel 0 of each owned patch row, -1 = zeros
#pragma unroll
            for (int i = 0; i < PPT; ++i) {
                const int pp = tid + i * LOADERS;
                src_off[i] = -1;
                if (pp < a.P) {
                    const long long g = gp0 + pp;
                    if (g >= 0 && g < a.total_pos) {
                        const long long b = g / a.Lp;
                        const int rem = (int)(g - b * a.Lp);
                        const int yy = rem / a.Wp, xx = rem - yy * a.Wp;
                        if (yy < a.H && xx < a.W) src_off[i] = b * a.C * a.HWin + (long long)(yy * a.stride) * a.Win + xx * a.stride;
                    }
                }
            }
            float va[PPT][CB], vb[PPT][CB];
            auto load = [&](int kb, float (&v)[PPT][CB]) {           // global -> registers, channel block kb
                const int c0 = kb * CB;
#pragma unroll
                for (int i = 0; i < PPT; ++i)
#pragma unroll
                    for (int j = 0; j < CB; ++j)
                        v[i][j] = (src_off[i] >= 0 && c0 + j < a.C) ? __ldg(a.x + src_off[i] + (long long)(c0 + j) * a.HWin) : 0.f;
            };
            auto stage = [&](int kb, float (&v)[PPT][CB]) -> bool {
                float* A = open_stage(kb);
                if (!A) return false;
#pragma unroll
                for (int i = 0; i < PPT; ++i) {
                    const int pp = tid + i * LOADERS;
                    if (pp < a.P) {
#pragma unroll
                        for (int q = 0; q < CB / 4; ++q) put(A, q, pp, v[i][4 * q], v[i][4 * q + 1], v[i][4 * q + 2], v[i][4 * q + 3]);
                    }
                }
                close_stage(kb);
                return true;
            };
            load(0, va);
            if (a.nkb > 1) load(1, vb);
            for (int kb = 0; kb < a.nkb; kb += 2) {
                if (!stage(kb, va)) break;
                if (kb + 2 < a.nkb) load(kb + 2, va);
                if (kb + 1 < a.nkb) {
                    if (!stage(kb + 1, vb)) break;
                    if (kb + 3 < a.nkb) load(kb + 3, vb);
                }
            }
        }
    } else {
        // ================= MMA issuers: warp 8+mt owns position tile mt =================
        const int mt = __shfl_sync(0xffffffffu, warp - 8, 0);
        if (mt < MT) {
            const uint32_t d_main = tmem + (uint32_t)(mt * a.tile_cols);
            int st_idx = 0, st_use = 0;
            for (int kb = 0; kb < a.nkb; ++kb) {
                const int s = st_idx;
                if (!mbar_wait(&full_bar[s], (uint32_t)st_use)) { *abort_flag = 1; break; }
                if (++st_idx == a.ns) { st_idx = 0; st_use ^= 1; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const float* A = stage0 + (long long)s * stage_floats;
                if (elect_one()) {
                    issue_block<NT, TAPS>(a, d_main, smem_u32(A), smem_u32(A + a_floats), (uint32_t)(mt * M_TILE), kb & 1, kb < 2 && (kb == 0 || a.nmain == 2));
                    mma_commit(&empty_bar[s]);
                    if (kb + 1 == a.nkb) mma_commit(done_bar);
                }
                __syncwarp();
            }
        }
    }

    // ---- epilogue: tensor memory -> registers -> y (NCHW: lanes = consecutive positions) ----
    __syncwarp();        // the issuing lane rejoins its warp before the CTA-wide barrier
    __syncthreads();
    bool fine = (*abort_flag == 0);
    if (fine) fine = mbar_wait(done_bar, 0);
    if (!fine) {
        if (a.status) atomicCAS(a.status, 0, 1);
    } else {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int q = warp & 3;                      // the lane quarter this warp may read
        constexpr int CHUNKS = NT / 32;
        for (int item = (warp >> 2); item < MT * CHUNKS; item += 3) {
            const int mt = item / CHUNKS, chunk = item - mt * CHUNKS;
            const long long g = g0 + mt * M_TILE + q * 32 + lane;
            long long out_off = -1;
            if (g < a.total_pos) {
                const long long b = g / a.Lp;
                const int rem = (int)(g - b * a.Lp);
                const int yy = rem / a.Wp, xx = rem - yy * a.Wp;
                if (yy < a.H && xx < a.W) out_off = b * a.K * HW + (long long)yy * a.W + xx;
            }
            uint32_t r[32];
            load_chunk<NT>(a, tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(mt * a.tile_cols + chunk * 32), r, a.nkb);
            store_chunk(a, r, out_off, ocb * NT + chunk * 32, HW);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 8) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

}  // namespace tdc_tc

#include "conv_tc_persist.cuh"

namespace tdc_tc {

// Filter [K][C][R][S] (or [C][R][S][K]) -> per (output block, channel block) the exact
// shared-memory image of a stage's B part: [tap][2 words][hl*NT rows][16 bytes] (rows 0..NT-1 the hi halves,
// NT..2NT-1 the lo halves of the same channels), zero-filled past C and K.  A 16-byte word holds 4 TF32 channels
// or, with f16, 8 fp16 channels (lo scaled by 2^11 like the input's).
// Largest magnitude of a tensor as ABSMAX_SLOTS partial maxima (no atomics, nothing to clear): block b writes entry
// b, block 0 zeroes the entries beyond the grid.  Magnitudes are compared as unsigned bit patterns.
__global__ void __launch_bounds__(256) absmax_kernel(const float* __restrict__ x, long long n, float* __restrict__ out) {
    __shared__ unsigned int red[8];
    unsigned int m = 0;
    const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
    if (reinterpret_cast<uintptr_t>(x) % 16 == 0) {
        const long long n4 = n >> 2;
        const uint4* x4 = reinterpret_cast<const uint4*>(x);
        auto take = [&](const uint4 v) { m = max(max(m, v.x & 0x7fffffffu), max(max(v.y & 0x7fffffffu, v.z & 0x7fffffffu), v.w & 0x7fffffffu)); };
        long long i = tid;
        for (; i + 7 * nthr < n4; i += 8 * nthr) {          // eight independent 16-byte loads in flight per thread
            uint4 v[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = __ldg(x4 + i + k * nthr);
#pragma unroll
            for (int k = 0; k < 8; ++k) take(v[k]);
        }
        for (; i < n4; i += nthr) take(__ldg(x4 + i));
        for (long long i = (n4 << 2) + tid; i < n; i += nthr) m = max(m, __float_as_uint(__ldg(x + i)) & 0x7fffffffu);
    } else {
        for (long long i = tid; i < n; i += nthr) m = max(m, __float_as_uint(__ldg(x + i)) & 0x7fffffffu);
    }
    m = __reduce_max_sync(0xffffffffu, m);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < 8; ++i) m = max(m, red[i]);
        out[blockIdx.x] = __uint_as_float(m);
    }
    if (blockIdx.x == 0)
        for (int i = gridDim.x + threadIdx.x; i < ABSMAX_SLOTS; i += blockDim.x) out[i] = 0.f;
}

__global__ void __launch_bounds__(256) prepare_weights_kernel(const float* __restrict__ w, int kcrs, float* __restrict__ wt, int C, int K, int taps,
                                       int nt, int nkb, int n_ocb, int hl, int f16, const float* __restrict__ w_absmax, float* __restrict__ w_scale,
                                       int row_S, int row_stride, int row_phase) {
    float ws = 1.f;                                           // fp16: the filter is scaled to the top of fp16's range
    if (f16) {
        __shared__ unsigned int word;
        ws = range_scale(absmax_of(w_absmax, &word));
        if (blockIdx.x == 0 && threadIdx.x == 0) *w_scale = ws;
    }
    const int epw = f16 ? 8 : 4;                              // elements per 16-byte word
    const long long per_block = (long long)hl * taps * 2 * epw * nt;
    const long long n = per_block * nkb * n_ocb;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        long long t = i;
        const int e = (int)(t % epw); t /= epw;
        const int nn = (int)(t % nt); t /= nt;
        const int h = (int)(t % hl); t /= hl;
        const int word = (int)(t % 2); t /= 2;
        const int tap = (int)(t % taps); t /= taps;
        const int kb = (int)(t % nkb); t /= nkb;
        const int ocb = (int)t;
        const int oc = ocb * nt + nn, c = (kb * 2 + word) * epw + e;
        float val = 0.f;
        if (row_stride) {
            // strided-row plan: channel c = (input channel, filter row) x column phase, tap = the filter's columns in steps of the stride
            const int cid = c / row_stride, dx = (tap - (row_phase ? 1 : 0)) * row_stride + c % row_stride + row_phase, Cr = C / row_stride;
            if (oc < K && c < C && dx >= 0 && dx < row_S) val = kcrs ? w[((long long)oc * Cr + cid) * row_S + dx] : w[((long long)cid * row_S + dx) * K + oc];
        } else if (oc < K && c < C) val = kcrs ? w[((long long)oc * C + c) * taps + tap] : w[((long long)c * taps + tap) * K + oc];
        if (f16) {
            val *= ws;
            const __half hi = __float2half_rn(val);
            reinterpret_cast<__half*>(wt)[i] = (h == 0) ? hi : __float2half_rn((val - __half2float(hi)) * 2048.f);
        } else {
            const float hi = to_tf32(val);
            wt[i] = (h == 0) ? hi : (val - hi);
        }
    }
}

}  // namespace tdc_tc

// ---------------------------------------------------------------------------------------------
#include "errors.h"

namespace {

using tdc::fail;
#define tc_fail fail
__device__ int g_tc_status;   // 0 = every wait of every launch so far completed

int pick_nt(int K) { return K > 64 ? 128 : (K > 32 ? 64 : 32); }

// What a launch would otherwise ask the runtime every time: per device the shared-memory limit, the SM count and
// the address of the status word; per (device, kernel) the dynamic shared-memory size already opted in.
struct DevFacts { int smem_max = 0, sms = 0; int* status = nullptr; };
std::mutex g_tc_mu;
std::map<int, DevFacts> g_tc_dev;
std::map<std::pair<int, const void*>, size_t> g_tc_smem_set;
int cdiv(int a, int b) { return (a + b - 1) / b; }

// Scratch behind a prepared fp16 filter: [0, ABSMAX_SLOTS) floats = partial maxima of |x| written by the range pass of
// the call in flight (calls that share a prepared filter must not overlap on the GPU), then one float = filter scale.
constexpr size_t TC_TAIL_BYTES = (tdc_tc::ABSMAX_SLOTS + 64) * sizeof(float);
float* tc_tail(const tdc_tc_plan* p, const void* wt) {
    return reinterpret_cast<float*>(reinterpret_cast<uintptr_t>(wt) + p->weights_bytes - TC_TAIL_BYTES);
}

// Tuning overrides.  They are measurement aids, not part of the interface: the environment is looked at only when
// TDC_TC_TUNING=1 was set before the first launch of the process, and then on every launch (tests switch them
// between calls); otherwise a launch reads no environment and its configuration is cached per layer shape.
//   TDC_TC_PERSIST 0/1 kernel, TDC_TC_MT cap on position tiles per CTA, TDC_TC_NS stages, TDC_TC_NBUF accumulator
//   buffers, TDC_TC_VEC 0/1 16-byte register loader of one-tap filters, TDC_TC_DEPTH raw slots, TDC_TC_KPS channel
//   blocks per stage (one-tap filters), TDC_TC_TAIL 0 = no smaller tiles in the last round, TDC_TC_CHAIN
//   accumulations per run (0 = one run), TDC_TC_BULK 0/1 bulk-tensor loader.
struct Tuning { int persist = -1, mt = -1, ns = -1, nbuf = -1, vec = -1, depth = -1, kps = -1, tail = -1, chain = -1, bulk = -1, pdl = -1, lw = -1; };
bool tuning_enabled() {
    static const bool on = [] { const char* v = getenv("TDC_TC_TUNING"); return v && atoi(v) != 0; }();
    return on;
}
Tuning read_tuning() {
    Tuning t;
    if (!tuning_enabled()) return t;
    auto get = [](const char* name) { const char* v = getenv(name); return v ? atoi(v) : -1; };
    t.persist = get("TDC_TC_PERSIST"); t.mt = get("TDC_TC_MT"); t.ns = get("TDC_TC_NS"); t.nbuf = get("TDC_TC_NBUF");
    t.vec = get("TDC_TC_VEC"); t.depth = get("TDC_TC_DEPTH"); t.kps = get("TDC_TC_KPS"); t.tail = get("TDC_TC_TAIL");
    t.chain = get("TDC_TC_CHAIN"); t.bulk = get("TDC_TC_BULK"); t.pdl = get("TDC_TC_PDL"); t.lw = get("TDC_TC_LW");
    return t;
}

// A launch, complete but for the pointers of the call.
struct Launch {
    tdc_tc::Args a;
    const void* fn = nullptr;
    const void* fn12 = nullptr;       // the same kernel with 12 loader warps and three epilogue groups (fp16 parts), or null
    unsigned ctas = 0;
    int threads = 0;
    size_t smem = 0;
    bool persist = false, bulk = false, pdl = false;
};
using LaunchKey = std::tuple<int, int, int, int, int, int, int, int, int, int, int, int, int>;
std::map<LaunchKey, Launch> g_tc_launches;

// cuTensorMapEncodeTiled, looked up through the runtime so that the library does not link against libcuda.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}

// Boxes the fullest raw slot of a launch needs: the patch of every position-tile start, with the rows of a full tile.
int max_boxes(int H, int W, int Wp, int Lp, long long total_pos, int mt, int halo_rows, int shift) {
    using namespace tdc_tc;
    const long long ptiles = (total_pos + M_TILE - 1) / M_TILE;
    // the pattern of image boundaries against tile starts repeats after lcm(Lp, 128) positions = Lp / gcd(Lp, 128) starts
    int g = Lp, h = M_TILE;
    while (h) { const int r = g % h; g = h; h = r; }
    const long long period = Lp / g + mt + 1;
    const long long scan = ptiles < period ? ptiles : period;
    int worst = 0;
    for (long long k = 0; k < scan; ++k) {
        const long long g0 = k * M_TILE, left = ptiles - k;
        const int rows = (int)(left < mt ? left : mt) * M_TILE + halo_rows;
        const long long gp0 = g0 - shift;
        const long long lo = gp0 < 0 ? 0 : gp0, hi = (gp0 + rows < total_pos ? gp0 + rows : total_pos) - 1;
        int nb = 0;
        for (long long b = lo / Lp; b <= hi / Lp; ++b) {
            int pix4, nbox;
            image_run(H, W, Wp, Lp, gp0, rows, b, pix4, nbox);
            nb += nbox;
        }
        if (nb > worst) worst = nb;
    }
    return worst;
}

}  // namespace

extern "C" {

const char* tdc_tc_last_error_string(void) { return tdc::last_error(); }

static int plan_fill(int C, int K, int R, int S, int mode, int general, tdc_tc_plan* out, int nt = 0, int stride = 0, int phase = 0) {
    if (!out) return tc_fail(TDC_ERR_NULL, "out is NULL");
    if (C <= 0 || K <= 0) return tc_fail(TDC_ERR_SHAPE, "C=%d K=%d", C, K);
    if (mode != 1 && mode != 3 && mode != 4) return tc_fail(TDC_ERR_UNSUPPORTED, "mode %d (1 = TF32, 3 = 3xTF32, 4 = 3xFP16)", mode);
    out->C = C; out->K = K; out->R = R; out->S = S; out->mode = mode;
    out->nt = nt ? nt : pick_nt(K);
    out->cb = mode == 4 ? 16 : 8;
    // a general plan contracts over (channel, filter row, filter column) triples, one tap; a strided-row plan over
    // (channel, filter row, column phase) triples, with the filter's columns in steps of the stride as taps
    out->stride = general == 2 ? stride : 0;
    out->phase = general == 2 ? phase : 0;
    const int taps_of = general == 2 ? cdiv(S + phase, stride) : (general ? 1 : R * S);
    out->nkb = cdiv(general == 2 ? C * R * stride : (general ? C * R * S : C), out->cb);
    out->n_ocb = cdiv(K, out->nt);
    out->hl = mode == 1 ? 1 : 2;
    out->general = general;
    // per (output block, channel block, tap): 32 bytes (one K step) for each of the hl * nt operand rows
    out->weights_bytes = sizeof(float) * (size_t)out->hl * taps_of * tdc_tc::CB * out->nt * out->nkb * out->n_ocb;
    // fp16 operands: a tail of scratch behind the filter holds the partial maxima of |x| of the call in flight and the
    // power of two the filter was scaled by (see tc_tail)
    if (mode == 4) out->weights_bytes += TC_TAIL_BYTES;
    return TDC_OK;
}

int tdc_tc_plan_make(int C, int K, int R, int S, int mode, tdc_tc_plan* out) {
    if (R != S || (R != 1 && R != 3))
        return tc_fail(TDC_ERR_UNSUPPORTED, "this plan is built for 1x1 and 3x3 filters, not %dx%d (tdc_tc_plan_make_general takes any)", R, S);
    return plan_fill(C, K, R, S, mode, 0, out);
}

int tdc_tc_pick_nt(int K, int mode, long long positions, int sm_count) {
    // Output channels per block for a layer with `positions` output positions (padding included): the default
    // (128 / 64 / 32 by K) serves layers whose tiles fill the SMs; with fewer tiles, smaller blocks give more CTAs.
    // Estimate per candidate: rounds of tiles over the SMs x clocks of one tap of one position tile and channel
    // block (the slower of the MMA pair's math and its operand reads from shared memory at 128 bytes per clock).
    if (K <= 0 || positions <= 0 || sm_count <= 0) return pick_nt(K > 0 ? K : 1);
    const int base = pick_nt(K);
    const long long ptiles = (positions + tdc_tc::M_TILE - 1) / tdc_tc::M_TILE;
    int best = base;
    double best_cost = 0.0;
    if (ptiles * ((K + base - 1) / base) >= sm_count) return base;      // every SM has a tile already
    for (int nt = base; nt >= 32; nt /= 2) {
        const double math = mode != 1 ? 96.0 * nt / 64.0 : 32.0 * nt / 64.0;
        const double smem = mode != 1 ? ((4096.0 + 64.0 * nt) + (4096.0 + 32.0 * nt)) / 128.0 : (4096.0 + 32.0 * nt) / 128.0;
        const long long tiles = ptiles * ((K + nt - 1) / nt);
        const double cost = (double)((tiles + sm_count - 1) / sm_count) * (math > smem ? math : smem);
        if (nt == base || cost < best_cost * 0.95) { best = nt; best_cost = cost; }      // a smaller block must win clearly
    }
    return best;
}

int tdc_tc_plan_make_nt(int C, int K, int R, int S, int mode, int general, int nt, tdc_tc_plan* out) {
    if (nt != 32 && nt != 64 && nt != 128) return tc_fail(TDC_ERR_UNSUPPORTED, "nt %d (32, 64 or 128)", nt);
    if (general) {
        if (R <= 0 || S <= 0 || R > 15 || S > 15) return tc_fail(TDC_ERR_SHAPE, "filter %dx%d", R, S);
        if ((long long)C * R * S > (1 << 20)) return tc_fail(TDC_ERR_SHAPE, "C*R*S = %lld is too long a contraction", (long long)C * R * S);
    } else if (R != S || (R != 1 && R != 3)) {
        return tc_fail(TDC_ERR_UNSUPPORTED, "this plan is built for 1x1 and 3x3 filters, not %dx%d", R, S);
    }
    return plan_fill(C, K, R, S, mode, general ? 1 : 0, out, nt);
}

// Column phase of a strided-row plan.  With stride 2 the loaders fetch both phases of a (channel, filter row) with one
// 8-byte copy, which must start on an even input column: the phases then count from column ox*2 - pad + phase with
// phase = pad mod 2, and the filter's first column becomes a tap of its own one position to the left (the plan keeps
// 2 or 4 taps for 3- and 7-wide filters; where the shift would add a tap the phase stays 0).
static int rows_phase(int S, int stride, int pad) {
    if (stride != 2 || !(pad & 1)) return 0;
    const int taps = cdiv(S + 1, 2);
    return (taps == 2 || taps == 4) ? 1 : 0;
}

int tdc_tc_plan_make_strided(int C, int K, int R, int S, int stride, int pad, int mode, int nt, tdc_tc_plan* out) {
    if (nt != 0 && nt != 32 && nt != 64 && nt != 128) return tc_fail(TDC_ERR_UNSUPPORTED, "nt %d (0, 32, 64 or 128)", nt);
    if (R <= 0 || S <= 0 || R > 15 || S > 15) return tc_fail(TDC_ERR_SHAPE, "filter %dx%d", R, S);
    if (stride < 2 || stride > 15) return tc_fail(TDC_ERR_UNSUPPORTED, "the strided-row plan is for strides 2..15, not %d", stride);
    if (pad < 0 || pad > 15) return tc_fail(TDC_ERR_UNSUPPORTED, "padding %d (0..15)", pad);
    const int phase = rows_phase(S, stride, pad);
    const int taps = cdiv(S + phase, stride);
    if (taps != 2 && taps != 4) return tc_fail(TDC_ERR_UNSUPPORTED, "the strided-row plan is built for 2 or 4 column taps (S/stride rounded up), not %d", taps);
    if (mode != 4) return tc_fail(TDC_ERR_UNSUPPORTED, "the strided-row plan is built for mode 4 (fp16 parts)");
    if ((long long)C * R * stride > (1 << 20)) return tc_fail(TDC_ERR_SHAPE, "C*R*stride = %lld is too long a contraction", (long long)C * R * stride);
    return plan_fill(C, K, R, S, mode, 2, out, nt, stride, phase);
}

int tdc_tc_plan_make_general(int C, int K, int R, int S, int mode, tdc_tc_plan* out) {
    if (R <= 0 || S <= 0 || R > 15 || S > 15) return tc_fail(TDC_ERR_SHAPE, "filter %dx%d", R, S);
    if ((long long)C * R * S > (1 << 20)) return tc_fail(TDC_ERR_SHAPE, "C*R*S = %lld is too long a contraction", (long long)C * R * S);
    return plan_fill(C, K, R, S, mode, 1, out);
}

int tdc_tc_prepare_weights(const tdc_tc_plan* p, const float* w, int w_layout, void* wt, void* stream) {
    if (!p || !w || !wt) return tc_fail(TDC_ERR_NULL, "plan, w and wt must be non-NULL");
    if (w_layout != TDC_W_KCRS && w_layout != TDC_W_CRSK) return tc_fail(TDC_ERR_UNSUPPORTED, "w_layout %d", w_layout);
    if (reinterpret_cast<uintptr_t>(wt) % 16 != 0) return tc_fail(TDC_ERR_UNSUPPORTED, "wt must be 16-byte aligned (the kernels fetch it with bulk copies)");
    const bool f16 = p->mode == 4;
    long long n = (long long)((p->weights_bytes - (f16 ? TC_TAIL_BYTES : 0)) / (f16 ? 2 : 4));
    int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
    float* tail = f16 ? tc_tail(p, wt) : nullptr;
    if (f16) {      // the filter's largest magnitude first: the prepare kernel scales by the power of two that follows from it
        const long long nw = (long long)p->C * p->K * p->R * p->S;
        tdc_tc::absmax_kernel<<<(unsigned)(nw / 1024 + 1 < 256 ? nw / 1024 + 1 : 256), 256, 0, (cudaStream_t)stream>>>(w, nw, tail);
    }
    // a general plan: the filter is a 1x1 filter over C*R*S channels; in both layouts channel, row and column are
    // adjacent index digits, so the flattened filter is addressed exactly as a 1x1 one
    const bool rows = p->general == 2;
    const int Cw = rows ? p->C * p->R * p->stride : (p->general ? p->C * p->R * p->S : p->C);
    const int taps = rows ? cdiv(p->S + p->phase, p->stride) : (p->general ? 1 : p->R * p->S);
    tdc_tc::prepare_weights_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(w, w_layout == TDC_W_KCRS, (float*)wt, Cw, p->K,
                                                                           taps, p->nt, p->nkb, p->n_ocb, p->hl, f16 ? 1 : 0, tail,
                                                                           tail ? tail + tdc_tc::ABSMAX_SLOTS : nullptr,
                                                                           rows ? p->S : 0, rows ? p->stride : 0, rows ? p->phase : 0);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? TDC_OK : tc_fail(TDC_ERR_CUDA, "prepare launch: %s", cudaGetErrorString(e));
}

// Everything about a launch that follows from the plan, the image and the flags: kernel, grid, shared memory and the
// argument block without its pointers.  `x_al16`: the input is 16-byte aligned (16-byte and bulk-tensor loads).
static int plan_launch(const tdc_tc_plan* p, int B, int H, int W, int flags, bool x_al16, const DevFacts& facts, const Tuning& tn, Launch* out) {
    using namespace tdc_tc;
    const int stride = (flags & TDC_TC_STRIDE_MASK) + 1, gpad = (flags & TDC_TC_PAD_MASK) >> TDC_TC_PAD_SHIFT;
    const bool f16 = p->mode == 4;
    const int cbk = f16 ? 16 : 8;
    Args a{};
    // from here on H and W are the output image; the input image is only an address pattern of the loaders
    a.stride = stride; a.Win = W; a.HWin = (long long)H * W; a.Hin = H;
    const int Hin = H, Win = W;
    if (p->general) {
        a.gather = 1; a.gR = p->R; a.gS = p->S; a.gpad = gpad; a.gpadx = gpad;
        if (H + 2 * gpad < p->R || W + 2 * gpad < p->S) return tc_fail(TDC_ERR_SHAPE, "the %dx%d filter does not fit the padded %dx%d image", p->R, p->S, H, W);
        H = (H + 2 * gpad - p->R) / stride + 1; W = (W + 2 * gpad - p->S) / stride + 1;
        if ((long long)p->C * a.HWin >= (1ll << 31)) return tc_fail(TDC_ERR_SHAPE, "channels x image = %lld elements is too large for a general plan", (long long)p->C * a.HWin);
    } else {
        H = (H - 1) / stride + 1; W = (W - 1) / stride + 1;
    }
    const bool rows = p->general == 2;            // strided-row plan
    const int taps_r = p->general ? 1 : p->R;     // filter size as the MMAs see it (one-pass plans)
    a.B = B; a.C = rows ? p->C * p->R * p->stride : (p->general ? p->C * p->R * p->S : p->C); a.H = H; a.W = W; a.K = p->K; a.taps_r = taps_r;
    const int pad = (taps_r - 1) / 2;
    const int taps = rows ? cdiv(p->S + p->phase, p->stride) : taps_r * taps_r;
    if (rows) {
        if (rows_phase(p->S, stride, gpad) != p->phase)
            return tc_fail(TDC_ERR_UNSUPPORTED, "this strided-row plan was made for a padding of the other parity than %d", gpad);
        a.gpadx = gpad - p->phase;
        // both phases of a (channel, filter row) are neighbours in memory: one 8-byte copy when they start on an even element
        a.gpair = (stride == 2 && Win % 2 == 0 && x_al16 && !(a.gpadx & 1)) ? 1 : 0;
        a.gS = p->stride;                 // the loaders' third index runs over the column phases, not the filter's columns
        a.Wp = W + taps - 1;              // a row of positions, then the taps' reach beyond it (gathered like any position)
        a.Lp = H * a.Wp;
        a.halo = taps - 1; a.shift = p->phase ? 1 : 0;     // with a phase the first tap looks one position to the left
    } else {
        a.Wp = W + pad;                       // one shared zero column per row when the filter has a halo
        a.Lp = (H + pad) * a.Wp;              // and one zero row after the image
        a.halo = 2 * pad * (a.Wp + 1); a.shift = pad * (a.Wp + 1);
    }
    a.total_pos = (long long)B * a.Lp;
    a.Hp = a.Lp / a.Wp;
    a.fd_Wp = fastdiv_make((uint32_t)a.Wp); a.fd_Lp = fastdiv_make((uint32_t)a.Lp);
    if (W > 256) return tc_fail(TDC_ERR_UNSUPPORTED, "image width %d is too large for the tensor-core path (max 256)", W);
    a.nkb = p->nkb; a.n_ocb = p->n_ocb; a.hl = p->hl;
    a.fd_nocb = fastdiv_make((uint32_t)a.n_ocb);
    const int smem_max = facts.smem_max, sms = facts.sms;
    // Long reductions get two main accumulators per tile, fed by even and odd channel blocks (4*NT columns per tile
    // instead of 2*NT): beyond 320 accumulations with TF32 operands, beyond 144 with fp16 operands (whose layers are
    // held closer to fp64); very long ones are cut into runs on top of that (below).
    a.nmain = (a.hl == 2 && (long long)p->nkb * taps > (f16 ? 144 : 320)) ? 2 : 1;
    a.tile_cols = (a.nmain == 2 ? 4 : 2) * p->nt;
    a.rz_unit = (a.hl == 2 && (flags & TDC_TC_UNBIASED)) ? 0x1p-26f * (float)taps / (float)a.nmain : 0.f;
    // The persistent kernel wins where a CTA tile is short and its prologue and epilogue would otherwise show: split
    // operands with up to 64 output channels per block, and one-tap filters of any block size (with few tiles too:
    // its cp.async ring has all loader threads and several channel blocks in flight, 20 % faster than the one-tile
    // kernel on nine layers of 25..200 tiles).  For 3x3 filters with 128-channel blocks and TF32 operands the one-tile
    // kernel, which drains tensor memory with all its warps, measured faster.  fp16 operands and general plans exist
    // in the persistent kernel only.
    const long long tiles_mt2 = ((a.total_pos + 2 * M_TILE - 1) / (2 * M_TILE)) * a.n_ocb;
    // ... and for 3x3 filters with one 128-channel block when the tile list has complete rounds plus a rest: the
    // persistent kernel spreads the rest over all SMs as smaller tiles (28x28x128 at batch 64: 88 -> 76 us).
    const bool persist = p->general || f16 || (tn.persist >= 0 ? tn.persist != 0
                                                    : (a.hl == 2 ? (p->nt <= 64 || taps == 1 || (tiles_mt2 >= sms && a.n_ocb == 1 && tiles_mt2 % sms != 0))
                                                                 // plain TF32: one-tap filters likewise (14 layers: 20 % on 12, level on 2); 3x3: two one-tile
                                                                 // CTAs share an SM for short launches, long ones measured faster persistent
                                                                 : (taps == 1 || 2.0 * a.total_pos * p->C * p->K * taps >= 8e9)));
    int mt = 512 / a.tile_cols > 4 ? 4 : 512 / a.tile_cols, ns = 0, depth = 0, nbuf = 1;   // tensor memory: 512 columns
    if (tn.mt >= 1) while (mt > tn.mt) mt /= 2;
    // 16-byte input loads: 1x1 filter, images a multiple of 4 positions long, 16-byte aligned base.  In the persistent
    // kernel the cp.async ring is the faster loader all the same — it keeps all 256 loader threads
    // and `depth` channel blocks in flight where the 16-byte path has 64 threads per 128-position tile and two blocks
    // in registers — except for blocks of up to 64 channels with ten or more position tiles per SM (157 one-tap
    // layers, 64..1024 -> 32..512 channels at 14..112 pixels, batch 1..128, timed both ways: ring/16-byte = 0.71-0.89
    // where the rule takes the ring, 1.06-1.14 where it does not; 0.88 geometric mean over all; plain TF32 on 14 of
    // them: the same picture).
    const bool vec_ok = !f16 && taps == 1 && !p->general && stride == 1 && ((long long)H * W) % 4 == 0 && x_al16;
    const long long ptiles = (a.total_pos + M_TILE - 1) / M_TILE;
    const bool ring_wins = persist && (p->nt > 64 || ptiles < 10ll * sms);
    const bool vec = vec_ok && (tn.vec >= 0 ? tn.vec != 0 : !ring_wins);
    // Bulk-tensor loader: fp16 operands, unit stride, the input image a multiple of 4 pixels (the stride of the
    // channel dimension of the tensor map must be a multiple of 16 bytes), 16-byte aligned input.
    const bool bulk_ok = f16 && !p->general && stride == 1 && ((long long)Hin * Win) % 4 == 0 && x_al16 && encode_tiled() != nullptr;
    bool bulk = bulk_ok && (tn.bulk >= 0 ? tn.bulk != 0 : true);
    // a warp computes the pixel runs of the images a patch meets one image per lane: at most 32 images per patch
    if (bulk && ((long long)2 * M_TILE + a.halo) / a.Lp + 2 > 32) bulk = false;
    const size_t header = persist ? P_HEADER : 128;
    const int halo_unit = a.halo;
    // Position tiles per CTA: the largest candidate (4, 2, 1; what tensor memory and shared memory hold) that still
    // gives every SM a tile.  One exception: when few position tiles share a large filter, streaming the filter
    // from L2 once per tile is what bounds the launch; then a larger candidate is taken if the estimate below
    // (shared-memory traffic at 128 bytes per clock per SM against filter bytes from L2) says it is faster.
    const double op_bytes = a.hl == 2 ? (4096.0 + 64.0 * p->nt) + (4096.0 + 32.0 * p->nt) : 4096.0 + 32.0 * p->nt;   // per tap and position tile
    const size_t room = (size_t)smem_max - header;
    auto raw_bytes_of = [&](int m, int P, bool use_bulk, int* cap) -> size_t {
        if (!persist || vec) return 0;
        if (!use_bulk) return sizeof(float) * (size_t)cbk * P;
        const int c = max_boxes(H, W, a.Wp, a.Lp, a.total_pos, m, halo_unit, a.shift);
        if (cap) *cap = c;
        return (size_t)c * BOXC * BOXW * sizeof(float);
    };
    // The bulk loader holds two position tiles per CTA at most.  Where the ring could hold four (blocks of 32 output
    // channels leave the shared memory for it) and there are tiles enough for that, the smaller share of halo rows wins:
    // 56x56x32 at batch 64: ring with four tiles 35.7 us, bulk with two 39.4 us; with blocks of 64 channels both hold
    // two and the bulk loader wins (56x56x64: 61 against 78 us).
    if (bulk && tn.bulk < 0 && mt >= 4 && taps == 9) {
        const int P4 = ((4 * M_TILE + halo_unit) + 7) / 8 * 8;
        const size_t sb4 = sizeof(float) * ((size_t)a.hl * CB * P4 + (size_t)a.hl * taps * CB * p->nt), rb4 = sizeof(float) * (size_t)cbk * P4;
        const long long tiles4 = ((a.total_pos + 4ll * M_TILE - 1) / (4ll * M_TILE)) * a.n_ocb;
        if (2 * sb4 + 2 * rb4 <= room && P4 <= p_rows_cap(4) && tiles4 >= sms) bulk = false;
    }
    if (bulk && mt > 2) mt = 2;                                 // its producer is the fourth issuer warp
    int best_mt = 0, big_mt = 0;
    double best_cost = 0.0, big_cost = 0.0;
    bool best_l2_bound = false;
    for (int attempt = 0; attempt < 2 && best_mt == 0; ++attempt) {
        if (attempt == 1) { if (!bulk) break; bulk = false; }     // the bulk loader's slots did not fit: fall back to the ring
        for (int m = mt; m >= 1; m /= 2) {
            const int P = ((m * M_TILE + halo_unit) + 7) / 8 * 8;
            const size_t sb = sizeof(float) * ((size_t)a.hl * CB * P + (size_t)a.hl * taps * CB * p->nt);
            int cap = 0;
            const size_t rb = raw_bytes_of(m, P, bulk, &cap);
            if (2 * sb + 2 * rb > room || P > (persist ? p_rows_cap(m) : 3 * LOADERS) || (bulk && (cap > P_MAXBOX || cap == 0))) continue;   // rows per loader thread the kernels are built for
            const double ntl = (double)((a.total_pos + (long long)m * M_TILE - 1) / ((long long)m * M_TILE)) * a.n_ocb;
            const double rounds = (double)(((long long)ntl + sms - 1) / sms);
            const double tile_clk = a.nkb * (m * taps * op_bytes + (double)sb + 2.0 * rb) / 128.0 + 2000.0 * m * (p->nt / 32);
            const double l2_clk = ntl * a.nkb * (double)(sizeof(float) * a.hl * taps * CB * p->nt) / 2900.0;
            const double cost = rounds * tile_clk > l2_clk ? rounds * tile_clk : l2_clk;
            if (big_mt == 0 || cost < big_cost) { big_mt = m; big_cost = cost; }          // cheapest of the candidates seen so far (all larger or equal)
            best_mt = m; best_cost = cost; best_l2_bound = l2_clk > rounds * tile_clk;
            if (ntl >= sms) break;
        }
    }
    if (best_mt != 0 && best_l2_bound && big_cost < best_cost) best_mt = big_mt;
    if (best_mt == 0) return tc_fail(TDC_ERR_SMEM, "two stages of the %dx%d filter block do not fit in shared memory", p->R, p->S);
    mt = best_mt;
    const bool ring = persist && !vec && !bulk;              // input staged through the raw cp.async ring
    // the persistent kernel double-buffers the accumulators when tensor memory has room for it
    if (persist && 2 * mt * a.tile_cols <= 512 && tn.nbuf != 1) nbuf = 2;
    a.P = ((mt * M_TILE + halo_unit) + 7) / 8 * 8;
    size_t stage_bytes = sizeof(float) * ((size_t)a.hl * CB * a.P + (size_t)a.hl * taps * CB * p->nt);
    int cap = 0;
    const size_t raw_bytes = raw_bytes_of(mt, a.P, bulk, &cap);
    a.nbox_cap = cap;
    // One-tap filters (1x1, general plans) do one or two MMAs per channel block and position tile: a stage of one
    // block would be all hand-over.  Their stages take up to four blocks (what leaves room for two stages and,
    // with a raw ring, two raw slots).
    a.kps = 1;
    if (persist && taps == 1) {
        int want = tn.kps >= 1 && tn.kps <= 8 ? tn.kps : 4;
        if (want > a.nkb) want = a.nkb;
        while (want > 1 && 2 * want * stage_bytes + 2 * raw_bytes > room) --want;
        a.kps = want;
        stage_bytes *= want;
    }
    if (ring || bulk) {
        // three operand stages when at least four raw slots still fit beside them, else two; then as many raw slots as fit
        ns = 3 * stage_bytes + 4 * raw_bytes <= room ? 3 : 2;
        if (tn.ns >= 2 && tn.ns <= 4 && tn.ns * stage_bytes + 2 * raw_bytes <= room) ns = tn.ns;
        depth = (int)((room - ns * stage_bytes) / raw_bytes);
        if (depth > 8) depth = 8;
        if (tn.depth >= 2 && tn.depth <= depth) depth = tn.depth;
    } else {
        const int ns_max = persist ? 4 : 3;
        ns = 2;
        while (ns < ns_max && (ns + 1) * stage_bytes <= room) ++ns;
        if (tn.ns >= 2 && tn.ns <= ns) ns = tn.ns;
    }
    if (!persist && ns > a.nkb) ns = a.nkb > 0 ? a.nkb : 1;
    a.ns = ns;
    a.nbuf = nbuf;
    a.depth = depth;
    a.tmem_cols = 32;
    while (a.tmem_cols < nbuf * mt * a.tile_cols) a.tmem_cols *= 2;
    // Runs: at most `chain` MMAs feed one accumulator before the epilogue takes the partial sum over in fp32.  The
    // error of the tensor core's running sum grows by about 2.5e-8 of the output scale per accumulation.  A run
    // boundary costs an extra pass of the epilogue over y (measured: about a microsecond per MB of y), so the default
    // only cuts reductions of more than 576 MMAs per output (3x3 filters over more than 1024 channels).
    a.nseg = 1; a.seg_blocks = a.nkb;
    const int chain = tn.chain >= 0 ? tn.chain : (f16 ? 288 : 0);
    if (persist && chain > 0) {
        const long long accs = ((long long)a.nkb * taps + a.nmain - 1) / a.nmain;
        int nseg = (int)((accs + chain - 1) / chain);
        if (nseg > 1) {
            int sb = cdiv(a.nkb, nseg);
            sb = cdiv(sb, a.kps) * a.kps;                   // a run ends with a stage
            a.seg_blocks = sb;
            a.nseg = cdiv(a.nkb, sb);
        }
    }
    const size_t smem = header + ns * stage_bytes + depth * raw_bytes;
    a.status = facts.status;
    long long tiles = (a.total_pos + (long long)mt * M_TILE - 1) / ((long long)mt * M_TILE);
    a.pt_total = (a.total_pos + M_TILE - 1) / M_TILE;
    a.full_groups = tiles; a.tail_first_pt = 0; a.tail_cnt = mt;          // every tile holds mt position tiles ...
    if (persist && a.n_ocb == 1 && mt > 1 && tn.tail != 0) {
        // ... except that the position tiles left for the last, partial round are spread over all SMs as smaller tiles
        const long long rounds = (a.pt_total / mt) / sms, full = rounds * sms, rest = a.pt_total - full * mt;
        if (rounds >= 1 && rest > 0) {          // (with no complete round the choice of mt above already weighed SMs against filter traffic)
            a.full_groups = full;
            a.tail_first_pt = full * mt;
            a.tail_cnt = (int)((rest + sms - 1) / sms);
            tiles = full + (rest + a.tail_cnt - 1) / a.tail_cnt;
        }
    }
    a.ntiles = tiles * a.n_ocb;
    a.small = a.total_pos + (long long)a.Lp + 4096 <= 0x7fffffffLL && a.ntiles <= 0x7fffffffLL;
    if (a.ntiles >= (1ll << 31)) return tc_fail(TDC_ERR_TILE, "grid too large");
    const long long ctas = persist ? (a.ntiles < sms ? a.ntiles : sms) : a.ntiles;
    // The persistent kernel with fp16 parts exists with 8 loader warps and four epilogue groups and with 12 and three;
    // which one a call takes depends on its epilogue and is decided per call (fn / fn_loaders below).  The TF32 kernels
    // exist with 8 only.
    const void *fn = nullptr, *fn12 = nullptr;
#define TDC_TC_ONE(NT_, MT_) (taps == 9 ? (const void*)&conv_tc_kernel<NT_, MT_, 9, false> : \
                              (vec ? (const void*)&conv_tc_kernel<NT_, MT_, 1, true> : (const void*)&conv_tc_kernel<NT_, MT_, 1, false>))
#define TDC_TC_PER(NT_, MT_, LW_) (f16 ? (taps == 9 ? (const void*)&conv_tc_persist_kernel<NT_, MT_, 9, LD_RING, true, LW_> \
                                          : taps == 4 ? (const void*)&conv_tc_persist_kernel<NT_, MT_, 4, LD_RING, true, LW_> \
                                          : taps == 2 ? (const void*)&conv_tc_persist_kernel<NT_, MT_, 2, LD_RING, true, LW_> \
                                                    : (const void*)&conv_tc_persist_kernel<NT_, MT_, 1, LD_RING, true, LW_>) \
                                       : (taps == 9 ? (const void*)&conv_tc_persist_kernel<NT_, MT_, 9, LD_RING, false> \
                                                    : (vec ? (const void*)&conv_tc_persist_kernel<NT_, MT_, 1, LD_VEC, false> \
                                                           : (const void*)&conv_tc_persist_kernel<NT_, MT_, 1, LD_RING, false>)))
#define TDC_TC_BLK(NT_, MT_, LW_) (taps == 9 ? (const void*)&conv_tc_persist_kernel<NT_, MT_, 9, LD_BULK, true, LW_> \
                                             : (const void*)&conv_tc_persist_kernel<NT_, MT_, 1, LD_BULK, true, LW_>)
#define TDC_TC_PICK(NT_, MT_, LW_) (persist ? TDC_TC_PER(NT_, MT_, LW_) : TDC_TC_ONE(NT_, MT_))
#define TDC_TC_ALL(LW_, FN_)                                                                                                     \
    if (bulk) {                                                                                                                  \
        if (p->nt == 128) FN_ = mt == 2 ? TDC_TC_BLK(128, 2, LW_) : TDC_TC_BLK(128, 1, LW_);                                     \
        else if (p->nt == 64) FN_ = mt == 2 ? TDC_TC_BLK(64, 2, LW_) : TDC_TC_BLK(64, 1, LW_);                                   \
        else FN_ = mt == 2 ? TDC_TC_BLK(32, 2, LW_) : TDC_TC_BLK(32, 1, LW_);                                                    \
    } else if (p->nt == 128) FN_ = mt == 2 ? TDC_TC_PICK(128, 2, LW_) : TDC_TC_PICK(128, 1, LW_);                                \
    else if (p->nt == 64) FN_ = mt == 4 ? TDC_TC_PICK(64, 4, LW_) : (mt == 2 ? TDC_TC_PICK(64, 2, LW_) : TDC_TC_PICK(64, 1, LW_)); \
    else FN_ = mt == 4 ? TDC_TC_PICK(32, 4, LW_) : (mt == 2 ? TDC_TC_PICK(32, 2, LW_) : TDC_TC_PICK(32, 1, LW_));
    TDC_TC_ALL(8, fn)
    if (persist && f16) { TDC_TC_ALL(12, fn12) }
#undef TDC_TC_ALL
#undef TDC_TC_PICK
#undef TDC_TC_BLK
#undef TDC_TC_PER
#undef TDC_TC_ONE
    if (tn.lw == 8) fn12 = nullptr;
    if (tn.lw == 12 && fn12) fn = fn12;
    out->fn12 = fn12;
    out->a = a; out->fn = fn; out->ctas = (unsigned)ctas; out->threads = persist ? P_THREADS : THREADS; out->smem = smem;
    out->persist = persist; out->bulk = bulk;
    out->pdl = persist && tn.pdl != 0;        // the persistent kernel waits for the grids before it on its own (griddepcontrol.wait)
    return TDC_OK;
}

int tdc_tc_check_launch(const tdc_tc_plan* p, int B, int H, int W, int flags) {
    if (!p) return tc_fail(TDC_ERR_NULL, "plan is NULL");
    if (B <= 0 || H <= 0 || W <= 0) return tc_fail(TDC_ERR_SHAPE, "B=%d H=%d W=%d", B, H, W);
    int device;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return tc_fail(TDC_ERR_NO_DEVICE, "cudaGetDevice: %s", cudaGetErrorString(e));
    DevFacts f;
    if ((e = cudaDeviceGetAttribute(&f.smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, device)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&f.sms, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess)
        return tc_fail(TDC_ERR_CUDA, "device query: %s", cudaGetErrorString(e));
    Launch L;
    return plan_launch(p, B, H, W, flags & ~TDC_TC_EXACT_RANGE, true, f, Tuning{}, &L);
}

int tdc_conv2d_tc(const tdc_tc_plan* p, const float* x, const void* wt, float* y, int B, int H, int W,
                  const tdc_epilogue* epi, int flags, void* stream) {
    return tdc_conv2d_tc_ranged(p, x, wt, y, B, H, W, epi, flags, nullptr, nullptr, stream);
}

int tdc_conv2d_tc_ranged(const tdc_tc_plan* p, const float* x, const void* wt, float* y, int B, int H, int W,
                         const tdc_epilogue* epi, int flags, const float* x_absmax, float* y_absmax, void* stream) {
    if (!p || !x || !wt || !y) return tc_fail(TDC_ERR_NULL, "plan, x, wt and y must be non-NULL");
    if (y_absmax && p->mode != 4) return tc_fail(TDC_ERR_UNSUPPORTED, "y_absmax is written by mode 4 (fp16 operands) only");
    if (B <= 0 || H <= 0 || W <= 0) return tc_fail(TDC_ERR_SHAPE, "B=%d H=%d W=%d", B, H, W);
    const int stride = (flags & TDC_TC_STRIDE_MASK) + 1, gpad = (flags & TDC_TC_PAD_MASK) >> TDC_TC_PAD_SHIFT;
    if (flags & ~(TDC_TC_STRIDE_MASK | TDC_TC_PAD_MASK | TDC_TC_EXACT_RANGE | TDC_TC_UNBIASED))
        return tc_fail(TDC_ERR_UNSUPPORTED, "unknown flag bits %#x", flags & ~(TDC_TC_STRIDE_MASK | TDC_TC_PAD_MASK | TDC_TC_EXACT_RANGE | TDC_TC_UNBIASED));
    if (!p->general && stride > 1 && p->R != 1) return tc_fail(TDC_ERR_UNSUPPORTED, "a stride is taken for 1x1 filters and general plans only");
    if (!p->general && gpad != 0) return tc_fail(TDC_ERR_UNSUPPORTED, "a padding is taken for general plans only (the others pad (R-1)/2)");
    if (p->general == 2 && stride != p->stride) return tc_fail(TDC_ERR_UNSUPPORTED, "this strided-row plan was made for stride %d, the call asks for %d", p->stride, stride);
    if (reinterpret_cast<uintptr_t>(wt) % 16 != 0) return tc_fail(TDC_ERR_UNSUPPORTED, "wt must be 16-byte aligned (the kernels fetch it with bulk copies)");
    using namespace tdc_tc;
    int device;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return tc_fail(TDC_ERR_NO_DEVICE, "cudaGetDevice: %s", cudaGetErrorString(e));
    DevFacts facts;
    {
        std::lock_guard<std::mutex> lk(g_tc_mu);
        auto it = g_tc_dev.find(device);
        if (it == g_tc_dev.end()) {
            DevFacts f;
            void* sp = nullptr;
            if ((e = cudaDeviceGetAttribute(&f.smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, device)) != cudaSuccess ||
                (e = cudaDeviceGetAttribute(&f.sms, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess ||
                (e = cudaGetSymbolAddress(&sp, g_tc_status)) != cudaSuccess)
                return tc_fail(TDC_ERR_CUDA, "device query: %s", cudaGetErrorString(e));
            f.status = (int*)sp;
            it = g_tc_dev.emplace(device, f).first;
        }
        facts = it->second;
    }
    const bool x_al16 = reinterpret_cast<uintptr_t>(x) % 16 == 0;
    Launch L;
    if (tuning_enabled()) {
        const int rc = plan_launch(p, B, H, W, flags & ~TDC_TC_EXACT_RANGE, x_al16, facts, read_tuning(), &L);
        if (rc) return rc;
    } else {
        const LaunchKey key{device, p->C, p->K, p->R, p->S, p->mode, p->nt, p->general, B, H, W, flags & ~TDC_TC_EXACT_RANGE, x_al16 ? 1 : 0};
        std::lock_guard<std::mutex> lk(g_tc_mu);
        auto it = g_tc_launches.find(key);
        if (it == g_tc_launches.end()) {
            const int rc = plan_launch(p, B, H, W, flags & ~TDC_TC_EXACT_RANGE, x_al16, facts, Tuning{}, &L);
            if (rc) return rc;
            it = g_tc_launches.emplace(key, L).first;
        }
        L = it->second;
    }
    Args& a = L.a;
    a.x = x; a.wt = (const float*)wt; a.y = y;
    if (epi) { a.scale = epi->scale; a.bias = epi->bias; a.residual = epi->residual; a.relu = epi->relu ? 1 : 0; }
    // The CTA's 28 warps: a launch whose epilogue only stores is paced by its loaders (12 loader warps, three epilogue
    // groups); one that scales, shifts, adds a residual or clamps wants the fourth epilogue group instead (8 loader warps).
    const void* fn_call = L.fn;
    int loader_threads = 256;
    if (L.fn12 && !(a.scale || a.bias || a.residual || a.relu)) { fn_call = L.fn12; loader_threads = 384; }
    if (L.fn12 && L.fn == L.fn12) loader_threads = 384;                 // forced by the tuning switch
    a.step_y = loader_threads / a.Wp; a.step_x = loader_threads % a.Wp;   // bulk loader: a thread's next row is this far on
    a.epi_vec = reinterpret_cast<uintptr_t>(a.scale) % 16 == 0 && reinterpret_cast<uintptr_t>(a.bias) % 16 == 0;
    if (p->mode == 4) {
        float* tail = tc_tail(p, wt);
        a.w_scale = tail + ABSMAX_SLOTS;
        a.y_absmax = y_absmax;
        a.x_absmax = x_absmax;
        a.x_count = (long long)B * p->C * H * W;
        if (!x_absmax && (flags & TDC_TC_EXACT_RANGE)) {
            // the caller wants the scale taken from the true maximum: one pass over the input first
            const long long n = a.x_count;
            const long long want = (n + 8191) / 8192;                      // 32 elements per thread at least
            const unsigned blocks = (unsigned)(want < 1 ? 1 : (want > 4 * facts.sms ? 4 * facts.sms : want));
            absmax_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(x, n, tail);
            if ((e = cudaGetLastError()) != cudaSuccess) return tc_fail(TDC_ERR_CUDA, "range pass launch: %s", cudaGetErrorString(e));
            a.x_absmax = tail;
        }
    }
    CUtensorMap tmap;
    memset(&tmap, 0, sizeof tmap);
    if (L.bulk) {
        // x as a 3-D tensor (pixels of an image, channels, images); a box is BOXW pixels of BOXC channels of one image
        const cuuint64_t gdim[3] = {(cuuint64_t)H * W, (cuuint64_t)p->C, (cuuint64_t)B};
        const cuuint64_t gstr[2] = {(cuuint64_t)H * W * sizeof(float), (cuuint64_t)p->C * H * W * sizeof(float)};
        const cuuint32_t box[3] = {(cuuint32_t)BOXW, (cuuint32_t)BOXC, 1u}, estr[3] = {1u, 1u, 1u};
        const CUresult r = encode_tiled()(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(x), gdim, gstr, box, estr,
                                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return tc_fail(TDC_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
    }
    {
        std::lock_guard<std::mutex> lk(g_tc_mu);
        size_t& have = g_tc_smem_set[{device, fn_call}];
        if (L.smem > have) {
            e = cudaFuncSetAttribute(fn_call, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L.smem);
            if (e != cudaSuccess) return tc_fail(TDC_ERR_CUDA, "cudaFuncSetAttribute(%zu): %s", L.smem, cudaGetErrorString(e));
            have = L.smem;
        }
    }
    void* args[] = {&a, &tmap};
    // Programmatic dependent launch: the persistent kernel may be scheduled while the kernel before it in the stream is
    // still running (its CTAs land on SMs as they become free, set up their barriers and tensor memory) and waits with
    // griddepcontrol.wait, which returns when every grid before it has completed and its writes are visible, before it
    // touches x, y or anything else a kernel before it may have written.  Only kernels launched with this attribute
    // start early, and every one of them waits; a kernel before or after without it is ordered as always.
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(L.ctas); cfg.blockDim = dim3(L.threads); cfg.dynamicSmemBytes = L.smem; cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = L.pdl ? 1 : 0;
    e = cudaLaunchKernelExC(&cfg, fn_call, args);
    return e == cudaSuccess ? TDC_OK : tc_fail(TDC_ERR_CUDA, "launch: %s", cudaGetErrorString(e));
}

#ifdef TDC_TC_PROFILE
// Measurement builds only: the 24 sums of the persistent kernel (see conv_tc_persist.cuh); reset != 0 clears them.
__attribute__((visibility("default"))) int tdc_tc_profile_read(unsigned long long* out, int reset) {
    cudaError_t e = cudaMemcpyFromSymbol(out, tdc_tc::g_tc_prof, sizeof(unsigned long long) * 24);
    if (e == cudaSuccess && reset) {
        unsigned long long z[24] = {};
        e = cudaMemcpyToSymbol(tdc_tc::g_tc_prof, z, sizeof z);
    }
    return e == cudaSuccess ? TDC_OK : tc_fail(TDC_ERR_CUDA, "profile read: %s", cudaGetErrorString(e));
}
#endif

int tdc_tc_status(int* out) {
    if (!out) return tc_fail(TDC_ERR_NULL, "out is NULL");
    cudaError_t e = cudaMemcpyFromSymbol(out, g_tc_status, sizeof(int));
    return e == cudaSuccess ? TDC_OK : tc_fail(TDC_ERR_CUDA, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
}

}  // extern "C"
