// Direct fp32 convolution for the core conv of a Tucker block (and the 1x1 convs
// around it), written for sm_100a.
//
// What the reference does for this step: inference/TKConv.py:92-93 calls
// F.conv2d(x, core_kernel, None, stride, padding); the CUDA artifact's kernel
// (A100-evaluation/TDC-LAYERS-ORACLE/template_benchmark_cudnn.template:365-402) gives
// each thread ONE output channel and a TH x TW patch of pixels, stages TC input
// channels of a row strip in shared memory, reads the nine weights of each channel
// from global memory, and sums channel chunks of different blocks with atomicAdd.
//
// What this kernel does instead:
//   * a thread owns TN output channels x (TH x TW) pixels in registers, so every
//     shared-memory word it loads feeds TN (input) or TH*TW (weight) FMAs;
//   * a CTA owns `nog*TN` output channels x a spatial tile of `imgs` images and walks
//     ALL input channels itself, chunk by chunk, so there is no atomicAdd and the
//     output needs no zeroing; the sum over channels has a fixed order;
//   * input patch (with its zero-padding halo) and the weight chunk are staged with
//     cp.async into a two-stage ring, the next chunk in flight while this one is used;
//   * the inner loop is shaped by the one resource that binds an fp32 direct conv on
//     this machine, the shared-memory return path (128 B per clock per SM against 128
//     FMAs per clock per SM): a channel's TN x 9 weights are read once into registers,
//     each staged input row is read once and used for every filter row it meets, and
//     the tallest thread tiles (TH = 4) reach ~12 FMAs per word loaded;
//   * the staged filter is laid out [tap][TN/4][NOG][4] so the eight lanes that share a
//     128-byte shared-memory wavefront read one contiguous, conflict-free line;
//   * `ks` thread slices may split the channels of a chunk (small feature maps leave
//     too few pixels to fill 148 SMs otherwise); slices are summed through shared
//     memory in slice order.
#pragma once
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tdc {

struct ConvArgs {
    const float* x;      // [B][C][H][W]
    const float* w;      // element (k,c,rs) at k*ws_k + c*ws_c + rs*ws_rs
    const float* bias;   // [K] or nullptr
    const float* scale;  // [K] or nullptr: y = conv * scale + bias (a folded BatchNorm)
    const float* residual;  // [B][K][Ho][Wo] or nullptr, added before the ReLU
    float*       y;      // [B][K][Ho][Wo]
    int B, C, H, W, K, Ho, Wo, pad;
    int R, S;            // filter size (used by the runtime-size variant only)
    long long ws_k, ws_c, ws_rs;
    int w_vec;           // 1: CRSK and K % 4 == 0 -> 16-byte weight copies
    int y_vec;           // 1: y is 16-byte aligned -> rows of a multiple of 4 outputs may be stored as 16-byte words
    int relu;
    // runtime part of the tile
    int tc, gy, gx, imgs, ks;
    int kc;              // CTAs of a cluster that share one output tile, each a range of chunks
    int chunks_per_rank;
    // derived by the host
    int in_rows, in_wp;  // rows / padded width of one image's staged input patch
    int patch;           // imgs * in_rows * in_wp, rounded up to a multiple of 4
    int tiles_y, tiles_x, img_groups, n_ocb;
    int stage_floats;    // floats of one stage (input part + weight part)
    // range-checked build (-DTDC_DEBUG_BOUNDS) only: element counts of x, w and y, and where a violation is recorded
    long long x_n, w_n, y_n;
    int* bounds;         // [0] violations seen, [1] kind of the first (1 x, 2 w, 3 y, 4 residual), [2..3] its offset
};

// Range-checked build: every global access of the kernel first checks its element offset against the tensor it
// belongs to; an access outside is not made, and the first one is recorded for the host (tdc_debug_bounds_read).
// This is the library's own stand-in for a memory checker: it finds an index error without faulting the GPU.
#ifdef TDC_DEBUG_BOUNDS
__device__ __forceinline__ bool bounds_ok(const ConvArgs& a, long long off, long long n, int kind) {
    if (off >= 0 && off < n) return true;
    if (a.bounds && atomicAdd(&a.bounds[0], 1) == 0) {
        a.bounds[1] = kind; a.bounds[2] = (int)(off & 0xffffffffll); a.bounds[3] = (int)(off >> 32);
    }
    return false;
}
#define TDC_BOUNDS(a, off, n, kind) bounds_ok(a, off, n, kind)
#else
#define TDC_BOUNDS(a, off, n, kind) true
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
// 4-byte async copy global->shared; `valid == false` writes a zero instead.
__device__ __forceinline__ void cp_async4(float* dst, const float* src, bool valid) {
    int sz = valid ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(sz)
                 : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src, bool valid) {
    int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(sz)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// Loads `LEN` consecutive floats. With VEC the address is 16-byte aligned by
// construction (window start = multiple of 4 floats in a row whose stride is a
// multiple of 4 floats).
template <int LEN, bool VEC>
__device__ __forceinline__ void load_window(const float* p, float (&v)[LEN]) {
    if constexpr (VEC) {
        constexpr int N4 = LEN / 4;
#pragma unroll
        for (int i = 0; i < N4; ++i) {
            float4 q = *reinterpret_cast<const float4*>(p + 4 * i);
            v[4 * i + 0] = q.x; v[4 * i + 1] = q.y; v[4 * i + 2] = q.z; v[4 * i + 3] = q.w;
        }
        constexpr int REM = LEN - 4 * N4;
        if constexpr (REM >= 2) {
            float2 q = *reinterpret_cast<const float2*>(p + 4 * N4);
            v[4 * N4] = q.x; v[4 * N4 + 1] = q.y;
        }
        if constexpr (REM == 1) v[4 * N4] = p[4 * N4];
        if constexpr (REM == 3) v[4 * N4 + 2] = p[4 * N4 + 2];
    } else {
#pragma unroll
        for (int i = 0; i < LEN; ++i) v[i] = p[i];
    }
}

// One tap's TN weights of this thread's channel group: float4 h of the group sits at
// (h*NOG + ocg)*4 in the tap's row; `p` already points at ocg*4.
template <int TN, int NOG>
__device__ __forceinline__ void load_taps(const float* p, float (&v)[TN]) {
#pragma unroll
    for (int h = 0; h < TN / 4; ++h) {
        float4 q = *reinterpret_cast<const float4*>(p + h * NOG * 4);
        v[4 * h + 0] = q.x; v[4 * h + 1] = q.y; v[4 * h + 2] = q.z; v[4 * h + 3] = q.w;
    }
}

// KH == 0 selects the runtime-size variant (any R,S up to 7, TH must be 1).
template <int KH, int KW, int STRIDE, int TN, int TH, int TW, int NOG, int MAXT>
__global__ void __launch_bounds__(MAXT) conv_f32_kernel(const ConvArgs a) {
    constexpr int OCB  = TN * NOG;
    constexpr int NACC = TN * TH * TW;
    constexpr bool RT  = (KH == 0);
    constexpr int ROWLEN = RT ? 1 : (TW - 1) * STRIDE + KW;
    constexpr bool VEC = !RT && ((TW * STRIDE) % 4 == 0);
    constexpr int CUNR = (KH * KW == 1) ? 4 : 1;   // 1x1: short body, unroll over channels

    extern __shared__ __align__(16) float smem[];
    int*   tab    = reinterpret_cast<int*>(smem);
    float* stages = smem + a.patch;

    const int R = RT ? a.R : KH, S = RT ? a.S : KW;
    const int RS = R * S;
    const int nthr = blockDim.x;
    const int tid  = threadIdx.x;

    // ---- which tile is this CTA ------------------------------------------------
    // The kc CTAs of a cluster are consecutive in blockIdx.x and work on the same tile.
    int bid = blockIdx.x / a.kc;
    const int crank = blockIdx.x - bid * a.kc;
    const int ocb = bid % a.n_ocb;  bid /= a.n_ocb;
    const int txi = bid % a.tiles_x; bid /= a.tiles_x;
    const int tyi = bid % a.tiles_y; bid /= a.tiles_y;
    const int b0  = bid * a.imgs;
    const int oc0 = ocb * OCB;
    const int oy0 = tyi * a.gy * TH;
    const int ox0 = txi * a.gx * TW;
    const long long HW = (long long)a.H * a.W;
    const float* xb = a.x + (long long)b0 * a.C * HW;

    // ---- which part of the tile is this thread -----------------------------------
    const int NT  = NOG * a.imgs * a.gy * a.gx;   // threads of one channel slice
    const int t   = tid % NT;
    const int ksl = tid / NT;
    const int ocg = t % NOG;
    int pg = t / NOG;
    const int gxi = pg % a.gx; pg /= a.gx;
    const int gyi = pg % a.gy;
    const int iml = pg / a.gy;
    const int win = (iml * a.in_rows + gyi * TH * STRIDE) * a.in_wp + gxi * TW * STRIDE;

    // ---- source-offset table of the staged patch (built once) ---------------------
    // Entry p = (image, patch row, patch column) -> offset of that input element from
    // xb for channel 0, or -1 where the patch lies in the zero padding / past the batch.
    {
        const int iy0 = oy0 * STRIDE - a.pad, ix0 = ox0 * STRIDE - a.pad;
        const int per_img = a.in_rows * a.in_wp;
        for (int p = tid; p < a.patch; p += nthr) {
            int im = p / per_img, rem = p - im * per_img;
            int iy = rem / a.in_wp, ix = rem - iy * a.in_wp;
            int yy = iy0 + iy, xx = ix0 + ix;
            bool ok = (im < a.imgs) && (b0 + im < a.B) && yy >= 0 && yy < a.H && xx >= 0 && xx < a.W;
            tab[p] = ok ? (int)((long long)im * a.C * HW + (long long)yy * a.W + xx) : -1;
        }
    }
    __syncthreads();

    const int in_stage = a.tc * a.patch;  // floats of the input part of a stage

    auto stage_chunk = [&](int c0, int tcc, float* st) {
        float* in_s = st;
        float* w_s  = st + in_stage;
        // input patch, one channel after another
        for (int cl = 0; cl < tcc; ++cl) {
            const float* src = xb + (long long)(c0 + cl) * HW;
            float* dst = in_s + cl * a.patch;
            for (int p = tid; p < a.patch; p += nthr) {
                int o = tab[p];
                const bool ok = o >= 0 && TDC_BOUNDS(a, (src - a.x) + o, a.x_n, 1);
                cp_async4(dst + p, src + (ok ? o : 0), ok);
            }
        }
        // weights of the chunk as [channel][r*S+s][OCB]
        if (a.w_vec) {
            constexpr int V = OCB / 4;
            const int items = tcc * RS * V;
            const float* src = a.w + ((long long)c0 * RS) * a.K + oc0;
            for (int i = tid; i < items; i += nthr) {
                int q = i / V, v = i - q * V;
                bool ok = (oc0 + 4 * v) < a.K;
                ok = ok && TDC_BOUNDS(a, (src - a.w) + (long long)q * a.K + 4 * v + 3, a.w_n, 2);
                int og = v / (TN / 4), h = v - og * (TN / 4);
                cp_async16(w_s + q * OCB + (h * NOG + og) * 4, src + (ok ? (long long)q * a.K + 4 * v : 0), ok);
            }
        } else {
            const int rows  = tcc * RS;
            const int items = rows * OCB;
            for (int i = tid; i < items; i += nthr) {
                int ol, q;
                if (a.ws_k == 1) { q = i / OCB; ol = i - q * OCB; }   // channel-last filter
                else             { ol = i / rows; q = i - ol * rows; } // torch filter: (c,r,s) contiguous
                int cl = q / RS, rs = q - cl * RS;
                bool ok = (oc0 + ol) < a.K;
                ok = ok && TDC_BOUNDS(a, (long long)(oc0 + ol) * a.ws_k + (long long)(c0 + cl) * a.ws_c + (long long)rs * a.ws_rs, a.w_n, 2);
                const float* src = a.w + (ok ? (long long)(oc0 + ol) * a.ws_k + (long long)(c0 + cl) * a.ws_c +
                                                   (long long)rs * a.ws_rs
                                             : 0);
                int og = ol / TN, rem = ol - og * TN;
                cp_async4(w_s + q * OCB + ((rem >> 2) * NOG + og) * 4 + (rem & 3), src, ok);
            }
        }
    };

    float acc[TN][TH][TW];
#pragma unroll
    for (int j = 0; j < TN; ++j)
#pragma unroll
        for (int o = 0; o < TH; ++o)
#pragma unroll
            for (int p = 0; p < TW; ++p) acc[j][o][p] = 0.f;

    const int nchunks_all = (a.C + a.tc - 1) / a.tc;
    const int kc_begin = crank * a.chunks_per_rank;
    const int nchunks  = min(nchunks_all, kc_begin + a.chunks_per_rank);   // this CTA walks [kc_begin, nchunks)
    if (kc_begin < nchunks) {
        stage_chunk(kc_begin * a.tc, min(a.tc, a.C - kc_begin * a.tc), stages);
        cp_async_commit();
    }

    for (int kc = kc_begin; kc < nchunks; ++kc) {
        float* cur = stages + ((kc - kc_begin) & 1) * a.stage_floats;
        if (kc + 1 < nchunks) {
            int c1 = (kc + 1) * a.tc;
            stage_chunk(c1, min(a.tc, a.C - c1), stages + ((kc + 1 - kc_begin) & 1) * a.stage_floats);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();

        const int tcc = min(a.tc, a.C - kc * a.tc);
        const float* in_s = cur + win;
        const float* w_s  = cur + in_stage + ocg * 4;

        if constexpr (!RT) {
            constexpr int IN_ROWS = (TH - 1) * STRIDE + KH;
#pragma unroll CUNR
            for (int cl = ksl; cl < tcc; cl += a.ks) {
                const float* ip = in_s + cl * a.patch;
                const float* wp = w_s + cl * (KH * KW * OCB);
                float wr[KH * KW][TN];
#pragma unroll
                for (int q = 0; q < KH * KW; ++q) load_taps<TN, NOG>(wp + q * OCB, wr[q]);
#pragma unroll
                for (int i = 0; i < IN_ROWS; ++i) {
                    float row[ROWLEN];
                    load_window<ROWLEN, VEC>(ip + i * a.in_wp, row);
#pragma unroll
                    for (int r = 0; r < KH; ++r) {
                        // input row i meets filter row r in output row o = (i - r) / STRIDE
                        if ((i - r) < 0 || (i - r) % STRIDE != 0 || (i - r) / STRIDE >= TH) continue;
                        const int o = (i - r) / STRIDE;
#pragma unroll
                        for (int s = 0; s < KW; ++s)
#pragma unroll
                            for (int j = 0; j < TN; ++j)
#pragma unroll
                                for (int p = 0; p < TW; ++p)
                                    acc[j][o][p] = fmaf(wr[r * KW + s][j], row[p * STRIDE + s], acc[j][o][p]);
                    }
                }
            }
        } else {
            for (int cl = ksl; cl < tcc; cl += a.ks) {
                const float* ip = in_s + cl * a.patch;
                const float* wp = w_s + cl * (RS * OCB);
                for (int r = 0; r < R; ++r)
                    for (int s = 0; s < S; ++s) {
                        float wv[TN];
                        load_taps<TN, NOG>(wp + (r * S + s) * OCB, wv);
                        const float* rp = ip + r * a.in_wp + s;
#pragma unroll
                        for (int p = 0; p < TW; ++p) {
                            float v = rp[p * STRIDE];
#pragma unroll
                            for (int j = 0; j < TN; ++j) acc[j][0][p] = fmaf(wv[j], v, acc[j][0][p]);
                        }
                    }
            }
        }
        __syncthreads();   // everyone is done with `cur` before the next prefetch overwrites it
    }

    // ---- sum the channel slices, slice 1 first, then 2, ... ---------------------------
    if (a.ks > 1) {
        float* red = stages;
        if (ksl > 0) {
#pragma unroll
            for (int j = 0; j < TN; ++j)
#pragma unroll
                for (int o = 0; o < TH; ++o)
#pragma unroll
                    for (int p = 0; p < TW; ++p)
                        red[((ksl - 1) * NACC + (j * TH + o) * TW + p) * NT + t] = acc[j][o][p];
        }
        __syncthreads();
        if (ksl == 0) {
            for (int k = 1; k < a.ks; ++k)
#pragma unroll
                for (int j = 0; j < TN; ++j)
#pragma unroll
                    for (int o = 0; o < TH; ++o)
#pragma unroll
                        for (int p = 0; p < TW; ++p)
                            acc[j][o][p] += red[((k - 1) * NACC + (j * TH + o) * TW + p) * NT + t];
        }
    }
    // ---- sum the CTAs of a cluster through distributed shared memory, rank 1 first --------
    if (a.kc > 1) {
        namespace cg = cooperative_groups;
        cg::cluster_group cluster = cg::this_cluster();
        float* red = stages;
        // slice 0 of every rank > 0 publishes its sums; a thread only overwrites entries that
        // it alone read in the slice reduction above, so no barrier is needed before this
        if (crank > 0 && ksl == 0) {
#pragma unroll
            for (int j = 0; j < TN; ++j)
#pragma unroll
                for (int o = 0; o < TH; ++o)
#pragma unroll
                    for (int p = 0; p < TW; ++p) red[((j * TH + o) * TW + p) * NT + t] = acc[j][o][p];
        }
        cluster.sync();
        if (crank == 0 && ksl == 0) {
            for (int r = 1; r < a.kc; ++r) {
                const float* peer = cluster.map_shared_rank(red, r);
#pragma unroll
                for (int j = 0; j < TN; ++j)
#pragma unroll
                    for (int o = 0; o < TH; ++o)
#pragma unroll
                        for (int p = 0; p < TW; ++p) acc[j][o][p] += peer[((j * TH + o) * TW + p) * NT + t];
            }
        }
        cluster.sync();   // peers keep their shared memory alive until rank 0 has read it
        if (crank != 0) return;
    }
    if (ksl != 0) return;

    // ---- epilogue: scale, bias, residual, ReLU, store ----------------------------------------------------
    const int b = b0 + iml;
    if (b >= a.B) return;
    const int oyb = oy0 + gyi * TH, oxb = ox0 + gxi * TW;
    const bool vec_st = a.y_vec && (a.Wo % 4 == 0);
#pragma unroll
    for (int j = 0; j < TN; ++j) {
        const int oc = oc0 + ocg * TN + j;
        if (oc >= a.K) continue;
        const float bv = a.bias ? a.bias[oc] : 0.f;
        const float sv = a.scale ? a.scale[oc] : 1.f;
        const long long plane = ((long long)b * a.K + oc) * a.Ho * a.Wo;
        float* yp = a.y + plane;
#pragma unroll
        for (int o = 0; o < TH; ++o) {
            const int oy = oyb + o;
            if (oy >= a.Ho) continue;
            float* yr = yp + (long long)oy * a.Wo + oxb;
#ifdef TDC_DEBUG_BOUNDS
            {   // the row this thread is about to write (and, with a residual, read): first and last element
                const int last = (oxb + TW <= a.Wo ? TW : a.Wo - oxb) - 1;
                if (last >= 0 && (!TDC_BOUNDS(a, (yr - a.y), a.y_n, 3) || !TDC_BOUNDS(a, (yr - a.y) + last, a.y_n, 3))) continue;
            }
#endif
#pragma unroll
            for (int p = 0; p < TW; ++p) {
                float v = a.scale ? fmaf(acc[j][o][p], sv, bv) : acc[j][o][p] + bv;
                if (a.residual && oxb + p < a.Wo) v += a.residual[plane + (long long)oy * a.Wo + oxb + p];
                acc[j][o][p] = a.relu ? fmaxf(v, 0.f) : v;
            }
            bool stored = false;
            if constexpr (TW % 4 == 0) {
                if (vec_st && oxb + TW <= a.Wo) {
#pragma unroll
                    for (int p = 0; p < TW; p += 4)
                        *reinterpret_cast<float4*>(yr + p) =
                            make_float4(acc[j][o][p], acc[j][o][p + 1], acc[j][o][p + 2], acc[j][o][p + 3]);
                    stored = true;
                }
            }
            if (!stored) {
#pragma unroll
                for (int p = 0; p < TW; ++p)
                    if (oxb + p < a.Wo) yr[p] = acc[j][o][p];
            }
        }
    }
}

}  // namespace tdc
