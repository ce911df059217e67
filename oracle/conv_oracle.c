/*
 * conv_oracle.c — CPU restatement of the reference's algorithm for the Tucker core
 * convolution.  TEST INFRASTRUCTURE ONLY: the tests, the smoke check and the benchmark's
 * CPU-baseline leg call it as the checker; nothing in the product may link or call it.
 *
 * What it restates
 *   (1) inference/TKConv.py:90-95  — TKConv2dC.forward: conv1x1, core conv with stride
 *       and zero padding, conv1x1 + bias.  The arithmetic of that file lives in
 *       torch.nn.functional.conv2d (PyTorch, "torch >= 1.4" per the reference README:16;
 *       2.11.0 in this image); what is restated here is its published definition,
 *       cross-correlation with zero padding:
 *         y[b][k][oy][ox] = sum_{c,r,s} x[b][c][oy*stride-pad+r][ox*stride-pad+s] * w[k][c][r][s]
 *   (2) A100-evaluation/TDC-LAYERS-ORACLE/template_benchmark_cudnn.template:340-402 — the
 *       CUDA kernel conv2d: blocks = channel chunks x row strips, a thread = one output
 *       channel x TH x TW pixels, partial sums of the chunks added into a zeroed output
 *       (tdc_oracle_conv2d_ref_tiled walks the blocks in blockIdx order).
 *
 * Pinning: the reference holds no golden tensors for this path.  This file is pinned by
 * (a) outputs of the reference's own TKConv2dC run on CPU, committed under tests/golden/
 * with the script that made them, and (b) the reference drivers' own check — integer
 * inputs 0..9 with all-ones weights give exact integers
 * (template_benchmark_cudnn.template:418-428,509).
 */
#include <math.h>
#include <pthread.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

/* ---- a small parallel-for over (image, output channel) pairs ------------------------
 * Threads: TDC_ORACLE_THREADS if set, else the online CPUs. Each pair is computed by
 * exactly one thread in a fixed arithmetic order, so results do not depend on the count. */
typedef void (*pair_fn)(int b, int k, void* ctx);
typedef struct { pair_fn fn; void* ctx; int K, n, tid, nthr; } pf_job;
static void* pf_run(void* p) {
    pf_job* j = (pf_job*)p;
    for (int i = j->tid; i < j->n; i += j->nthr) j->fn(i / j->K, i % j->K, j->ctx);
    return NULL;
}
int tdc_oracle_threads(void) {
    const char* e = getenv("TDC_ORACLE_THREADS");
    long n = e ? atol(e) : sysconf(_SC_NPROCESSORS_ONLN);
    return n < 1 ? 1 : (n > 256 ? 256 : (int)n);
}
static void parallel_pairs(int B, int K, pair_fn fn, void* ctx) {
    int n = B * K, nthr = tdc_oracle_threads();
    if (nthr > n) nthr = n;
    if (nthr <= 1) { for (int i = 0; i < n; ++i) fn(i / K, i % K, ctx); return; }
    pthread_t th[256]; pf_job jobs[256];
    for (int t = 0; t < nthr; ++t) {
        jobs[t] = (pf_job){fn, ctx, K, n, t, nthr};
        pthread_create(&th[t], NULL, pf_run, &jobs[t]);
    }
    for (int t = 0; t < nthr; ++t) pthread_join(th[t], NULL);
}
typedef struct {
    const float *x, *w, *bias; float* y;
    int B, C, H, W, K, R, S, pad, stride, w_layout, use_fma, relu, tc, ks, kc;
} conv_ctx;

#define W_KCRS 0
#define W_CRSK 1

static inline size_t widx(int layout, int K, int C, int R, int S, int k, int c, int r, int s) {
    if (layout == W_KCRS) return (((size_t)k * C + c) * R + r) * S + s;
    return (((size_t)c * R + r) * S + s) * K + k;
}

/* fp32 accumulation in the order c, r, s (ascending), one fused multiply-add per tap
 * when use_fma != 0, a rounded product and a rounded sum otherwise. Padding taps are
 * skipped (adding 0*w changes nothing for finite w). */
#define UNPACK(q) \
    const conv_ctx* q_ = (const conv_ctx*)(q); const float *x = q_->x, *w = q_->w, *bias = q_->bias; float* y = q_->y; \
    const int C = q_->C, H = q_->H, W = q_->W, K = q_->K, R = q_->R, S = q_->S, pad = q_->pad, stride = q_->stride, \
              w_layout = q_->w_layout, relu = q_->relu; \
    const int Ho = (H + 2 * pad - R) / stride + 1, Wo = (W + 2 * pad - S) / stride + 1;

static void f32_pair(int b, int k, void* q) {
    UNPACK(q)
    const int use_fma = q_->use_fma;
            for (int oy = 0; oy < Ho; ++oy)
                for (int ox = 0; ox < Wo; ++ox) {
                    float acc = 0.f;
                    for (int c = 0; c < C; ++c)
                        for (int r = 0; r < R; ++r) {
                            int iy = oy * stride - pad + r;
                            if (iy < 0 || iy >= H) continue;
                            for (int s = 0; s < S; ++s) {
                                int ix = ox * stride - pad + s;
                                if (ix < 0 || ix >= W) continue;
                                float xv = x[(((size_t)b * C + c) * H + iy) * W + ix];
                                float wv = w[widx(w_layout, K, C, R, S, k, c, r, s)];
                                if (use_fma) acc = fmaf(wv, xv, acc);
                                else { volatile float p = wv * xv; acc = acc + p; }
                            }
                        }
                    if (bias) acc += bias[k];
                    if (relu && acc < 0.f) acc = 0.f;
                    y[(((size_t)b * K + k) * Ho + oy) * Wo + ox] = acc;
                }
}
void tdc_oracle_conv2d_f32(const float* x, const float* w, const float* bias, float* y, int B, int C, int H,
                           int W, int K, int R, int S, int pad, int stride, int w_layout, int use_fma, int relu) {
    conv_ctx c = {x, w, bias, y, B, C, H, W, K, R, S, pad, stride, w_layout, use_fma, relu, 0, 0, 1};
    parallel_pairs(B, K, f32_pair, &c);
}

/* Same sum in the order the CUDA kernel uses when a CTA splits each staged chunk of
 * `tc` channels over `ks` slices: slice j owns channels j, j+ks, ... of every chunk and
 * sums them (c, r, s ascending, fmaf, padding taps included as +0*w which leaves the
 * value unchanged); then the slices are added 0 + 1 + 2 + ...; when the chunks are split
 * over the kc CTAs of a cluster, each CTA does that for its range of chunks and the CTAs
 * are added in rank order.  Bit-exact twin of the device result for that (tc, ks, kc). */
static void sliced_pair(int b, int k, void* q) {
    UNPACK(q)
    const int tc = q_->tc, ks = q_->ks, kc = q_->kc;
    const int nchunks = (C + tc - 1) / tc, cpr = (nchunks + kc - 1) / kc;
            for (int oy = 0; oy < Ho; ++oy)
                for (int ox = 0; ox < Wo; ++ox) {
                    float total = 0.f;
                    for (int rank = 0; rank < kc; ++rank) {            /* CTAs of a cluster, rank order */
                        float rsum = 0.f;
                        for (int j = 0; j < ks; ++j) {                 /* slices of a CTA, slice order   */
                            float acc = 0.f;
                            for (int ch = rank * cpr; ch < (rank + 1) * cpr && ch < nchunks; ++ch)
                                for (int c = ch * tc + j; c < (ch + 1) * tc && c < C; c += ks)
                                    for (int r = 0; r < R; ++r)
                                        for (int s = 0; s < S; ++s) {
                                            int iy = oy * stride - pad + r, ix = ox * stride - pad + s;
                                            float xv = (iy < 0 || iy >= H || ix < 0 || ix >= W)
                                                           ? 0.f
                                                           : x[(((size_t)b * C + c) * H + iy) * W + ix];
                                            acc = fmaf(w[widx(w_layout, K, C, R, S, k, c, r, s)], xv, acc);
                                        }
                            rsum = (j == 0) ? acc : rsum + acc;
                        }
                        total = (rank == 0) ? rsum : total + rsum;
                    }
                    if (bias) total += bias[k];
                    if (relu) total = fmaxf(total, 0.f);
                    y[(((size_t)b * K + k) * Ho + oy) * Wo + ox] = total;
                }
}
void tdc_oracle_conv2d_f32_sliced(const float* x, const float* w, const float* bias, float* y, int B, int C,
                                  int H, int W, int K, int R, int S, int pad, int stride, int w_layout, int tc,
                                  int ks, int kc, int relu) {
    conv_ctx c = {x, w, bias, y, B, C, H, W, K, R, S, pad, stride, w_layout, 1, relu, tc, ks, kc};
    parallel_pairs(B, K, sliced_pair, &c);
}

/* The arbiter: double accumulation, rounded to float once. */
static void f64_pair(int b, int k, void* q) {
    UNPACK(q)
            for (int oy = 0; oy < Ho; ++oy)
                for (int ox = 0; ox < Wo; ++ox) {
                    double acc = 0.0;
                    for (int c = 0; c < C; ++c)
                        for (int r = 0; r < R; ++r) {
                            int iy = oy * stride - pad + r;
                            if (iy < 0 || iy >= H) continue;
                            for (int s = 0; s < S; ++s) {
                                int ix = ox * stride - pad + s;
                                if (ix < 0 || ix >= W) continue;
                                acc += (double)x[(((size_t)b * C + c) * H + iy) * W + ix] *
                                       (double)w[widx(w_layout, K, C, R, S, k, c, r, s)];
                            }
                        }
                    if (bias) acc += (double)bias[k];
                    if (relu && acc < 0.0) acc = 0.0;
                    y[(((size_t)b * K + k) * Ho + oy) * Wo + ox] = (float)acc;
                }
}
void tdc_oracle_conv2d_f64(const float* x, const float* w, const float* bias, float* y, int B, int C, int H,
                           int W, int K, int R, int S, int pad, int stride, int w_layout, int relu) {
    conv_ctx c = {x, w, bias, y, B, C, H, W, K, R, S, pad, stride, w_layout, 0, relu, 0, 0, 1};
    parallel_pairs(B, K, f64_pair, &c);
}

/*
 * The reference CUDA kernel conv2d (template_benchmark_cudnn.template:365-402) walked on
 * the CPU, block by block in blockIdx order, thread by thread:
 *   grid  = TCS*THS blocks, tile_id -> (tc_id = tile_id / THS, th_id = tile_id % THS)  (:367-369)
 *   block = N*TWS threads, thread -> (tw_id = tid / N, n = tid % N)                    (:370-374)
 *   shared strip [TC][TH+2][WPAD] zeroed, rows h_out_start-1 .. filled at column +1    (:377-388, :340-363)
 *   per channel: nine weights k[c][r][s][n], TH*TW partial sums                        (:390-400)
 *   write-back: atomicAdd of min(TH,H-h0) x min(TW,W-w0) values into outputs[n][h][w]  (:401)
 * 3x3, pad 1, stride 1, one image, filter layout [C][3][3][N], outputs must start at 0.
 * Requires C % TC == 0 like the reference (no channel bound check there).
 */
int tdc_oracle_conv2d_ref_tiled(const float* input, const float* kernel, float* outputs, int C, int N, int H,
                                int W, int TH, int TW, int TC) {
    if (C % TC) return 1;
    const int TCS = (C - 1) / TC + 1, THS = (H - 1) / TH + 1, TWS = (W - 1) / TW + 1, WPAD = TWS * TW + 2;
    float* sh = (float*)malloc(sizeof(float) * TC * (TH + 2) * WPAD);
    float* acc = (float*)malloc(sizeof(float) * TH * TW);
    if (!sh || !acc) { free(sh); free(acc); return 2; }
    for (int tile_id = 0; tile_id < TCS * THS; ++tile_id) {
        const int tc_id = tile_id / THS, th_id = tile_id % THS;
        const int h_out_start = th_id * TH, c_offset = tc_id * TC;
        const int h_offset = (h_out_start == 0) ? 1 : 0;
        const int h_padded_end = (h_out_start + TH + 2 < H + 2) ? h_out_start + TH + 2 : H + 2;
        const int h_start = (h_out_start - 1 > 0) ? h_out_start - 1 : 0;
        const int h_end = (H < h_padded_end - 1) ? H : h_padded_end - 1;
        memset(sh, 0, sizeof(float) * TC * (TH + 2) * WPAD);
        for (int c = 0; c < TC; ++c)
            for (int i = 0; i < (h_end - h_start) * W; ++i) {
                int r = i / W, s = i % W;
                sh[c * (TH + 2) * WPAD + (h_offset + r) * WPAD + s + 1] = input[(size_t)(c_offset + c) * H * W + h_start * W + i];
            }
        for (int tw_id = 0; tw_id < TWS; ++tw_id)
            for (int n = 0; n < N; ++n) {
                const int w_out_start = tw_id * TW;
                for (int i = 0; i < TH * TW; ++i) acc[i] = 0.f;
                for (int c = 0; c < TC; ++c)
                    for (int h = 0; h < TH + 2; ++h)
                        for (int w = 0; w < TW + 2; ++w) {
                            float v = sh[c * (TH + 2) * WPAD + h * WPAD + tw_id * TW + w];
                            for (int r = 0; r < 3; ++r)
                                for (int s = 0; s < 3; ++s) {
                                    int oh = h - r, ow = w - s;
                                    if (oh < 0 || oh >= TH || ow < 0 || ow >= TW) continue;
                                    acc[oh * TW + ow] += v * kernel[(size_t)(c + c_offset) * N * 9 + r * 3 * N + s * N + n];
                                }
                        }
                const int wh = (TH < H - h_out_start) ? TH : H - h_out_start;
                const int ww = (TW < W - w_out_start) ? TW : W - w_out_start;
                for (int th = 0; th < wh; ++th)
                    for (int tw = 0; tw < ww; ++tw)
                        outputs[(size_t)n * H * W + (h_out_start + th) * W + (w_out_start + tw)] += acc[th * TW + tw];
            }
    }
    free(sh); free(acc);
    return 0;
}

/* TKConv2dC.forward (inference/TKConv.py:90-95) from the three convs above; z1 and z2 are
 * caller-provided scratch of B*R1*H*W and B*R2*Ho*Wo floats. f64 != 0 selects the arbiter. */
void tdc_oracle_tk_block(const float* x, const float* w1, const float* wcore, const float* w3, const float* bias,
                         float* y, float* z1, float* z2, int B, int C, int H, int W, int R1, int R2, int K, int R,
                         int S, int pad, int stride, int core_layout, int f64) {
    const int Ho = (H + 2 * pad - R) / stride + 1, Wo = (W + 2 * pad - S) / stride + 1;
    if (f64) {
        tdc_oracle_conv2d_f64(x, w1, NULL, z1, B, C, H, W, R1, 1, 1, 0, 1, W_KCRS, 0);
        tdc_oracle_conv2d_f64(z1, wcore, NULL, z2, B, R1, H, W, R2, R, S, pad, stride, core_layout, 0);
        tdc_oracle_conv2d_f64(z2, w3, bias, y, B, R2, Ho, Wo, K, 1, 1, 0, 1, W_KCRS, 0);
    } else {
        tdc_oracle_conv2d_f32(x, w1, NULL, z1, B, C, H, W, R1, 1, 1, 0, 1, W_KCRS, 1, 0);
        tdc_oracle_conv2d_f32(z1, wcore, NULL, z2, B, R1, H, W, R2, R, S, pad, stride, core_layout, 1, 0);
        tdc_oracle_conv2d_f32(z2, w3, bias, y, B, R2, Ho, Wo, K, 1, 1, 0, 1, W_KCRS, 1, 0);
    }
}
