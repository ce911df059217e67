// cuDNN baselines of the per-shape layer drivers: the three algorithm classes the reference times beside its kernel
// (ConvGemm / ConvWinogradeNon / ConvFFT = cudnnConvolutionForward with CUDNN_CONVOLUTION_FWD_ALGO_IMPLICIT_GEMM,
// _WINOGRAD and _FFT; A100-evaluation/TDC-LAYERS-ORACLE/template_benchmark_cudnn.template:49-340, timed at :455-477).
// A measurement tool, not part of libtdc_b200.so: it links cuDNN and runs in a process of its own, so that the
// cuDNN it loads is never mixed with the one a Python process already holds.
//
//   cudnn_layer_baseline B C H W K R S pad stride [iters]
//
// Input rand()%10 with a fixed seed, filter all ones, fp32 NCHW — the reference's tensors and descriptors — with
// CUDNN_FMA_MATH, so that no algorithm converts to TF32.  Prints one line
//   fft_ms,winograd_ms,gemm_ms,fft_diff,winograd_diff
// where a time is the median of `iters` launches after one warm-up launch (the reference times one launch after one
// warm-up), `nan` where cuDNN does not support the algorithm for the shape on this GPU, and the diffs are the L1
// distance of that algorithm's output to the implicit-GEMM output (the reference's check_diff).
#include <cuda_runtime.h>
#include <cudnn.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#define CK(call)                                                                         \
    do {                                                                                 \
        cudaError_t e_ = (call);                                                         \
        if (e_ != cudaSuccess) {                                                         \
            std::fprintf(stderr, "%s: %s\n", #call, cudaGetErrorString(e_));             \
            return 2;                                                                    \
        }                                                                                \
    } while (0)
#define DNN(call)                                                                        \
    do {                                                                                 \
        cudnnStatus_t s_ = (call);                                                       \
        if (s_ != CUDNN_STATUS_SUCCESS) {                                                \
            std::fprintf(stderr, "%s: %s\n", #call, cudnnGetErrorString(s_));            \
            return 2;                                                                    \
        }                                                                                \
    } while (0)

struct Layer {
    cudnnHandle_t h;
    cudnnTensorDescriptor_t xd, yd;
    cudnnFilterDescriptor_t wd;
    cudnnConvolutionDescriptor_t cd;
    const float *x, *w;
    float* y;
};

// Median time of one algorithm in ms, or NaN when cuDNN refuses it; its output stays in L.y.
static double time_algo(const Layer& L, cudnnConvolutionFwdAlgo_t algo, int iters) {
    size_t ws_bytes = 0;
    if (cudnnGetConvolutionForwardWorkspaceSize(L.h, L.xd, L.wd, L.cd, L.yd, algo, &ws_bytes) != CUDNN_STATUS_SUCCESS) return NAN;
    void* ws = nullptr;
    if (ws_bytes && cudaMalloc(&ws, ws_bytes) != cudaSuccess) { cudaGetLastError(); return NAN; }
    const float one = 1.f, zero = 0.f;
    auto run = [&]() { return cudnnConvolutionForward(L.h, &one, L.xd, L.x, L.wd, L.w, L.cd, algo, ws, ws_bytes, &zero, L.yd, L.y); };
    double result = NAN;
    if (run() == CUDNN_STATUS_SUCCESS && cudaDeviceSynchronize() == cudaSuccess) {
        cudaEvent_t e0, e1;
        cudaEventCreate(&e0); cudaEventCreate(&e1);
        std::vector<float> ts;
        for (int i = 0; i < iters; ++i) {
            cudaEventRecord(e0);
            if (run() != CUDNN_STATUS_SUCCESS) break;
            cudaEventRecord(e1);
            cudaEventSynchronize(e1);
            float ms = 0.f;
            cudaEventElapsedTime(&ms, e0, e1);
            ts.push_back(ms);
        }
        if ((int)ts.size() == iters) { std::sort(ts.begin(), ts.end()); result = ts[ts.size() / 2]; }
        cudaEventDestroy(e0); cudaEventDestroy(e1);
    }
    if (ws) cudaFree(ws);
    return result;
}

static double l1(const std::vector<float>& a, const std::vector<float>& b) {
    double d = 0;
    for (size_t i = 0; i < a.size(); ++i) d += std::fabs((double)a[i] - (double)b[i]);
    return d;
}

int main(int argc, char** argv) {
    if (argc < 10) {
        std::fprintf(stderr, "usage: %s B C H W K R S pad stride [iters]\n", argv[0]);
        return 1;
    }
    const int B = atoi(argv[1]), C = atoi(argv[2]), H = atoi(argv[3]), W = atoi(argv[4]), K = atoi(argv[5]), R = atoi(argv[6]),
              S = atoi(argv[7]), pad = atoi(argv[8]), stride = atoi(argv[9]), iters = argc > 10 ? atoi(argv[10]) : 20;
    if (B <= 0 || C <= 0 || H <= 0 || W <= 0 || K <= 0 || R <= 0 || S <= 0 || pad < 0 || stride <= 0 || iters <= 0) return 1;
    Layer L{};
    DNN(cudnnCreate(&L.h));
    DNN(cudnnCreateTensorDescriptor(&L.xd));
    DNN(cudnnCreateTensorDescriptor(&L.yd));
    DNN(cudnnCreateFilterDescriptor(&L.wd));
    DNN(cudnnCreateConvolutionDescriptor(&L.cd));
    DNN(cudnnSetTensor4dDescriptor(L.xd, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, B, C, H, W));
    DNN(cudnnSetFilter4dDescriptor(L.wd, CUDNN_DATA_FLOAT, CUDNN_TENSOR_NCHW, K, C, R, S));
    DNN(cudnnSetConvolution2dDescriptor(L.cd, pad, pad, stride, stride, 1, 1, CUDNN_CROSS_CORRELATION, CUDNN_DATA_FLOAT));
    DNN(cudnnSetConvolutionMathType(L.cd, CUDNN_FMA_MATH));       // fp32 arithmetic: no TF32 down-conversion
    int ob, ok, oh, ow;
    DNN(cudnnGetConvolution2dForwardOutputDim(L.cd, L.xd, L.wd, &ob, &ok, &oh, &ow));
    DNN(cudnnSetTensor4dDescriptor(L.yd, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, ob, ok, oh, ow));
    const size_t nx = (size_t)B * C * H * W, nw = (size_t)K * C * R * S, ny = (size_t)ob * ok * oh * ow;
    std::vector<float> hx(nx), hw(nw, 1.0f);
    srand(1);
    for (auto& v : hx) v = (float)(rand() % 10);
    float *dx, *dw;
    CK(cudaMalloc(&dx, nx * 4)); CK(cudaMalloc(&dw, nw * 4)); CK(cudaMalloc(&L.y, ny * 4));
    CK(cudaMemcpy(dx, hx.data(), nx * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dw, hw.data(), nw * 4, cudaMemcpyHostToDevice));
    L.x = dx; L.w = dw;

    std::vector<float> ref(ny), out(ny);
    const double gemm = time_algo(L, CUDNN_CONVOLUTION_FWD_ALGO_IMPLICIT_GEMM, iters);
    CK(cudaMemcpy(ref.data(), L.y, ny * 4, cudaMemcpyDeviceToHost));
    double t[2], d[2];
    const cudnnConvolutionFwdAlgo_t algos[2] = {CUDNN_CONVOLUTION_FWD_ALGO_FFT, CUDNN_CONVOLUTION_FWD_ALGO_WINOGRAD};
    for (int i = 0; i < 2; ++i) {
        CK(cudaMemset(L.y, 0, ny * 4));
        t[i] = time_algo(L, algos[i], iters);
        d[i] = NAN;
        if (!std::isnan(t[i]) && !std::isnan(gemm)) {
            CK(cudaMemcpy(out.data(), L.y, ny * 4, cudaMemcpyDeviceToHost));
            d[i] = l1(out, ref);
        }
    }
    std::printf("%f,%f,%f,%g,%g\n", t[0], t[1], gemm, d[0], d[1]);
    cudaFree(dx); cudaFree(dw); cudaFree(L.y);
    cudnnDestroyConvolutionDescriptor(L.cd); cudnnDestroyFilterDescriptor(L.wd);
    cudnnDestroyTensorDescriptor(L.xd); cudnnDestroyTensorDescriptor(L.yd); cudnnDestroy(L.h);
    return 0;
}
