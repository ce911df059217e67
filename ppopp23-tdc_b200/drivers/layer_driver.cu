// Per-shape layer driver, native: the counterpart of the program the reference generates for every shape
// (A100-evaluation/TDC-LAYERS-ORACLE/template_benchmark_cudnn.template:404-514, built and run per shape by
// compile_run.py:14-52).  As there, main() fills the input with rand() % 10 and the filter with ones, times the
// kernel with a cudaEvent pair around one un-warmed launch, checks the result with an L1 difference that must be
// exactly 0 for these integers, prints one CSV row and appends it to a file.  Unlike there, shape and tile are
// arguments (the reference's macros may still be given with -D, as LAYER_C, LAYER_N, ..., and become the defaults),
// the kernel comes from libtdc_b200.so through its C ABI, the expected output is computed on the host (all-ones
// weights make it a windowed sum of the input over all channels), and a warmed median is reported beside the first launch.
//
//   layer_driver C N H W [--batch B] [--filter K] [--stride S] [--pad P] [--tile th,tw,tc,tn,nog,gy,gx,imgs,ks,kc]
//                [--tc 0|1|3|4] [--iters n] [--csv file] [--reference-row]
//
// C = input channels, N = output channels of the core conv (the reference's naming).
// Row: N,C,H,W,B,first_ms,median_ms,frac_fp32,diff   or, with --reference-row, the reference's own columns
// N,C,H,W,FFT,WINO,GEMM,TVM,TDC,FFT/TDC,WINO/TDC,GEMM/TDC,TVM/TDC,diff (template_benchmark_cudnn.template:500-512),
// the cuDNN columns taken from the cudnn_layer_baseline tool beside this program (nan when it is absent), TVM nan.
#include <cuda_runtime.h>
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>
#include "tdc_b200.h"

// Compile-time defaults, the reference's macros under prefixed names (a bare C, N, H or W would rename fields of the
// library's own header): -DLAYER_C=64 -DLAYER_N=64 -DLAYER_H=56 -DLAYER_W=56 [-DLAYER_TH=.. -DLAYER_TW=.. -DLAYER_TC=..]
#ifndef LAYER_C
#define LAYER_C 0
#endif
#ifndef LAYER_N
#define LAYER_N 0
#endif
#ifndef LAYER_H
#define LAYER_H 0
#endif
#ifndef LAYER_W
#define LAYER_W 0
#endif
#ifndef LAYER_TH
#define LAYER_TH 0
#endif
#ifndef LAYER_TW
#define LAYER_TW 0
#endif
#ifndef LAYER_TC
#define LAYER_TC 0
#endif

namespace {

struct Options {
    int c = LAYER_C, n = LAYER_N, h = LAYER_H, w = LAYER_W, batch = 1, filter = 3, stride = 1, pad = 1, tc = 0, iters = 20;
    bool reference_row = false;
    tdc_tile tile{LAYER_TH, LAYER_TW, LAYER_TC, 0, 0, 0, 0, 0, 0, 0};
    std::string csv;
};

int usage(const char* argv0) {
    fprintf(stderr, "usage: %s C N H W [--batch B] [--filter K] [--stride S] [--pad P] [--tile th,tw,tc,tn,nog,gy,gx,imgs,ks,kc] "
                    "[--tc 0|1|3|4] [--iters n] [--csv file] [--reference-row]\n", argv0);
    return 2;
}

bool cuda_ok(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return true;
    fprintf(stderr, "layer_driver: %s: %s\n", what, cudaGetErrorString(e));
    return false;
}

// The reference's check_diff (template_benchmark_cudnn.template:404-411): sum of absolute differences.
double check_diff(const float* x, const float* y, size_t size) {
    double diff = 0.0;
    for (size_t i = 0; i < size; ++i) diff += std::fabs((double)x[i] - (double)y[i]);
    return diff;
}

// cuDNN's three algorithm classes for this layer from the baseline tool, a process of its own.
void cudnn_columns(const char* argv0, const Options& o, double* fft, double* wino, double* gemm) {
    *fft = *wino = *gemm = NAN;
    std::string dir(argv0);
    const size_t slash = dir.find_last_of('/');
    dir = slash == std::string::npos ? "." : dir.substr(0, slash);
    char cmd[1024];
    snprintf(cmd, sizeof cmd, "%s/cudnn_layer_baseline %d %d %d %d %d %d %d %d %d %d 2>/dev/null", dir.c_str(), o.batch, o.c, o.h, o.w,
             o.n, o.filter, o.filter, o.pad, o.stride, o.iters);
    FILE* p = popen(cmd, "r");
    if (!p) return;
    double a, b, c;
    if (fscanf(p, "%lf,%lf,%lf", &a, &b, &c) == 3) { *fft = a; *wino = b; *gemm = c; }
    pclose(p);
}

}  // namespace

int main(int argc, char** argv) {
    Options o;
    std::vector<const char*> pos;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        auto next = [&]() -> const char* { return i + 1 < argc ? argv[++i] : ""; };
        if (a == "--batch") o.batch = atoi(next());
        else if (a == "--filter") o.filter = atoi(next());
        else if (a == "--stride") o.stride = atoi(next());
        else if (a == "--pad") o.pad = atoi(next());
        else if (a == "--tc") o.tc = atoi(next());
        else if (a == "--iters") o.iters = atoi(next());
        else if (a == "--csv") o.csv = next();
        else if (a == "--reference-row") o.reference_row = true;
        else if (a == "--tile") {
            int v[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
            sscanf(next(), "%d,%d,%d,%d,%d,%d,%d,%d,%d,%d", v, v + 1, v + 2, v + 3, v + 4, v + 5, v + 6, v + 7, v + 8, v + 9);
            o.tile = tdc_tile{v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7], v[8], v[9]};
        } else if (a.rfind("--", 0) == 0) return usage(argv[0]);
        else pos.push_back(argv[i]);
    }
    if (pos.size() == 4) { o.c = atoi(pos[0]); o.n = atoi(pos[1]); o.h = atoi(pos[2]); o.w = atoi(pos[3]); }
    else if (!pos.empty()) return usage(argv[0]);
    if (o.c <= 0 || o.n <= 0 || o.h <= 0 || o.w <= 0 || o.batch <= 0 || o.iters <= 0) return usage(argv[0]);
    if (o.tc != 0 && o.tc != 1 && o.tc != 3 && o.tc != 4) return usage(argv[0]);

    const int k = o.filter, ho = (o.h + 2 * o.pad - k) / o.stride + 1, wo = (o.w + 2 * o.pad - k) / o.stride + 1;
    if (ho <= 0 || wo <= 0) { fprintf(stderr, "layer_driver: empty output\n"); return 2; }
    const size_t in_n = (size_t)o.batch * o.c * o.h * o.w, out_n = (size_t)o.batch * o.n * ho * wo, w_n = (size_t)o.c * k * k * o.n;
    std::vector<float> input(in_n), ones(w_n, 1.0f), out(out_n), expect(out_n);
    srand(1);
    for (size_t i = 0; i < in_n; ++i) input[i] = (float)(rand() % 10);
    // all-ones weights: every output channel is the windowed sum of the input over all channels
    std::vector<float> chan_sum((size_t)o.batch * o.h * o.w, 0.f);
    for (int b = 0; b < o.batch; ++b)
        for (int c = 0; c < o.c; ++c)
            for (int i = 0; i < o.h * o.w; ++i) chan_sum[(size_t)b * o.h * o.w + i] += input[((size_t)b * o.c + c) * o.h * o.w + i];
    for (int b = 0; b < o.batch; ++b)
        for (int y = 0; y < ho; ++y)
            for (int x = 0; x < wo; ++x) {
                float s = 0.f;
                for (int r = 0; r < k; ++r)
                    for (int q = 0; q < k; ++q) {
                        const int iy = y * o.stride - o.pad + r, ix = x * o.stride - o.pad + q;
                        if (iy >= 0 && iy < o.h && ix >= 0 && ix < o.w) s += chan_sum[((size_t)b * o.h + iy) * o.w + ix];
                    }
                for (int n = 0; n < o.n; ++n) expect[(((size_t)b * o.n + n) * ho + y) * wo + x] = s;
            }

    float *d_in = nullptr, *d_w = nullptr, *d_out = nullptr;
    void* d_wt = nullptr;
    if (!cuda_ok(cudaMalloc((void**)&d_in, in_n * 4), "cudaMalloc") || !cuda_ok(cudaMalloc((void**)&d_w, w_n * 4), "cudaMalloc") ||
        !cuda_ok(cudaMalloc((void**)&d_out, out_n * 4), "cudaMalloc"))
        return 1;
    cudaMemcpy(d_in, input.data(), in_n * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(d_w, ones.data(), w_n * 4, cudaMemcpyHostToDevice);      // [c][r][s][n], the reference kernel's layout; all ones
    cudaMemset(d_out, 0, out_n * 4);

    tdc_tc_plan plan{};
    if (o.tc) {
        int rc = (o.stride == 1 && o.pad == (k - 1) / 2 && (k == 1 || k == 3)) ? tdc_tc_plan_make(o.c, o.n, k, k, o.tc, &plan)
                                                                              : tdc_tc_plan_make_general(o.c, o.n, k, k, o.tc, &plan);
        if (rc) { fprintf(stderr, "layer_driver: %s\n", tdc_last_error_string()); return 1; }
        if (!cuda_ok(cudaMalloc(&d_wt, plan.weights_bytes), "cudaMalloc")) return 1;
        if ((rc = tdc_tc_prepare_weights(&plan, d_w, TDC_W_CRSK, d_wt, nullptr))) { fprintf(stderr, "layer_driver: %s\n", tdc_last_error_string()); return 1; }
    }
    const int flags = o.tc ? ((o.stride - 1) | (plan.general ? (o.pad << TDC_TC_PAD_SHIFT) : 0)) : 0;
    tdc_tile tile_arg = o.tile;
    auto launch = [&]() -> int {
        if (o.tc) return tdc_conv2d_tc(&plan, d_in, d_wt, d_out, o.batch, o.h, o.w, nullptr, flags, nullptr);
        return tdc_core_conv2d_f32(d_in, d_w, d_out, o.batch, o.c, o.h, o.w, o.n, k, k, o.pad, o.stride, TDC_W_CRSK, &tile_arg, nullptr);
    };
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    auto timed = [&](float* ms) -> int {
        cudaEventRecord(e0);
        const int rc = launch();
        cudaEventRecord(e1);
        cudaEventSynchronize(e1);
        cudaEventElapsedTime(ms, e0, e1);
        return rc;
    };
    float first_ms = 0.f;
    if (timed(&first_ms)) { fprintf(stderr, "layer_driver: %s\n", tdc_last_error_string()); return 1; }     // the reference's protocol: one launch, not warmed
    if (!cuda_ok(cudaDeviceSynchronize(), "kernel")) return 1;
    for (int i = 0; i < 3; ++i) launch();
    std::vector<float> ts(o.iters);
    for (int i = 0; i < o.iters; ++i) timed(&ts[i]);
    std::sort(ts.begin(), ts.end());
    const double tdc_ms = ts[o.iters / 2];
    cudaMemcpy(out.data(), d_out, out_n * 4, cudaMemcpyDeviceToHost);
    const double diff = check_diff(out.data(), expect.data(), out_n);
    int tc_status = 0;
    if (o.tc) tdc_tc_status(&tc_status);

    tdc_devinfo dev;
    tdc_query_device(-1, &dev);
    const double flops = 2.0 * o.batch * o.n * o.c * k * k * ho * wo;
    const double frac = flops / (tdc_ms * 1e-3) / (dev.sm_count * 128.0 * 2.0 * 1.965e9);
    char row[1024];
    if (o.reference_row) {
        double fft, wino, gemm;
        cudnn_columns(argv[0], o, &fft, &wino, &gemm);
        const double tvm = NAN;
        snprintf(row, sizeof row, "%d,%d,%d,%d,%f,%f,%f,%f,%f,%f,%f,%f,%f,%g", o.n, o.c, o.h, o.w, fft, wino, gemm, tvm, tdc_ms, fft / tdc_ms,
                 wino / tdc_ms, gemm / tdc_ms, tvm / tdc_ms, diff);
    } else {
        snprintf(row, sizeof row, "%d,%d,%d,%d,%d,%f,%f,%f,%g", o.n, o.c, o.h, o.w, o.batch, first_ms, tdc_ms, frac, diff);
    }
    printf("%s\n", row);
    if (!o.csv.empty()) {
        FILE* f = fopen(o.csv.c_str(), "a");
        if (!f) { fprintf(stderr, "layer_driver: cannot open %s\n", o.csv.c_str()); return 1; }
        fprintf(f, "%s\n", row);
        fclose(f);
    }
    cudaFree(d_in); cudaFree(d_w); cudaFree(d_out); cudaFree(d_wt);
    return (diff == 0.0 && tc_status == 0) ? 0 : 1;
}
