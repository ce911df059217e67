// Pooling layer of the end-to-end skeleton: the reference's Pool::initialize(b,c,h,w,pad,windowH,windowW,
// mode,stride) / Pool::forward (A100-evaluation/EndToEnd/resnet18-tk/src/Pool.cu:8-48, a cudnnPoolingForward
// call) and the nn.MaxPool2d(3, 2, 1) after the stem (inference/resnet_inet_tt.py:323,384).  Memory-bound:
// every input element is read once from HBM (neighbouring windows overlap in cache), every output written once.
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>
#include "../../include/tdc_b200.h"
#include "errors.h"

namespace {

// One thread per output element, lanes along the output row.
__global__ void pool_generic_kernel(const float* __restrict__ x, float* __restrict__ y, long long planes, int H, int W, int Ho,
                                    int Wo, int kh, int kw, int pad, int stride, int mode) {
    const long long n = planes * Ho * Wo;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int ox = (int)(i % Wo), oy = (int)((i / Wo) % Ho);
        const float* xp = x + (i / ((long long)Wo * Ho)) * H * W;
        const int y0 = oy * stride - pad, x0 = ox * stride - pad;
        float m = -FLT_MAX, s = 0.f;
        int cnt = 0;
        for (int r = 0; r < kh; ++r) {
            const int iy = y0 + r;
            if ((unsigned)iy >= (unsigned)H) continue;
            for (int c = 0; c < kw; ++c) {
                const int ix = x0 + c;
                if ((unsigned)ix >= (unsigned)W) continue;
                const float v = __ldg(xp + (long long)iy * W + ix);
                m = fmaxf(m, v); s += v; ++cnt;
            }
        }
        y[i] = mode == TDC_POOL_MAX ? m : (mode == TDC_POOL_AVG_INCLUDE_PAD ? s / (float)(kh * kw) : s / (float)(cnt > 0 ? cnt : 1));
    }
}

// 3x3 window, stride 2, pad 1, max, W a multiple of 8: a thread makes 4 neighbouring outputs from the 9 input
// columns 8t-1 .. 8t+7 of three rows — two aligned 16-byte loads and one scalar per row, one 16-byte store.
__global__ void maxpool_3x3s2_kernel(const float* __restrict__ x, float* __restrict__ y, long long planes, int H, int W, int Ho, int Wo) {
    const int q = Wo / 4;                                    // threads per output row
    const long long n = planes * Ho * q;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i % q), oy = (int)((i / q) % Ho);
        const long long plane = i / ((long long)q * Ho);
        const float* xp = x + plane * H * W;
        float o0 = -FLT_MAX, o1 = -FLT_MAX, o2 = -FLT_MAX, o3 = -FLT_MAX;
#pragma unroll
        for (int r = 0; r < 3; ++r) {
            const int iy = 2 * oy - 1 + r;
            if ((unsigned)iy >= (unsigned)H) continue;
            const float* row = xp + (long long)iy * W + 8 * t;
            const float4 a = __ldg(reinterpret_cast<const float4*>(row));
            const float4 b = __ldg(reinterpret_cast<const float4*>(row + 4));
            const float l = t > 0 ? __ldg(row - 1) : -FLT_MAX;
            o0 = fmaxf(o0, fmaxf(l, fmaxf(a.x, a.y)));
            o1 = fmaxf(o1, fmaxf(a.y, fmaxf(a.z, a.w)));
            o2 = fmaxf(o2, fmaxf(a.w, fmaxf(b.x, b.y)));
            o3 = fmaxf(o3, fmaxf(b.y, fmaxf(b.z, b.w)));
        }
        *reinterpret_cast<float4*>(y + (plane * Ho + oy) * Wo + 4 * t) = make_float4(o0, o1, o2, o3);
    }
}

// 2x2 window, stride 2, no padding, max (the pooling of the VGG feature stack, inference/vgg_tt.py:116-123), H even,
// W a multiple of 8: a thread makes 4 neighbouring outputs from two aligned 16-byte loads in each of two rows.
__global__ void maxpool_2x2s2_kernel(const float* __restrict__ x, float* __restrict__ y, long long planes, int H, int W, int Ho, int Wo) {
    const int q = Wo / 4;
    const long long n = planes * Ho * q;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i % q), oy = (int)((i / q) % Ho);
        const long long plane = i / ((long long)q * Ho);
        const float* row = x + plane * H * W + (long long)(2 * oy) * W + 8 * t;
        const float4 a0 = __ldg(reinterpret_cast<const float4*>(row)), b0 = __ldg(reinterpret_cast<const float4*>(row + 4));
        const float4 a1 = __ldg(reinterpret_cast<const float4*>(row + W)), b1 = __ldg(reinterpret_cast<const float4*>(row + W + 4));
        *reinterpret_cast<float4*>(y + (plane * Ho + oy) * Wo + 4 * t) =
            make_float4(fmaxf(fmaxf(a0.x, a0.y), fmaxf(a1.x, a1.y)), fmaxf(fmaxf(a0.z, a0.w), fmaxf(a1.z, a1.w)),
                        fmaxf(fmaxf(b0.x, b0.y), fmaxf(b1.x, b1.y)), fmaxf(fmaxf(b0.z, b0.w), fmaxf(b1.z, b1.w)));
    }
}

}  // namespace

extern "C" int tdc_pool2d_f32(const float* x, float* y, int B, int C, int H, int W, int window_h, int window_w, int pad,
                              int stride, int mode, void* stream) {
    using tdc::fail;
    if (!x || !y) return fail(TDC_ERR_NULL, "tdc_pool2d_f32: x and y must be non-NULL");
    if (B <= 0 || C <= 0 || H <= 0 || W <= 0 || window_h <= 0 || window_w <= 0 || pad < 0 || stride <= 0)
        return fail(TDC_ERR_SHAPE, "tdc_pool2d_f32: B=%d C=%d H=%d W=%d window %dx%d pad=%d stride=%d", B, C, H, W, window_h, window_w, pad, stride);
    if (mode != TDC_POOL_MAX && mode != TDC_POOL_AVG_INCLUDE_PAD && mode != TDC_POOL_AVG_EXCLUDE_PAD)
        return fail(TDC_ERR_UNSUPPORTED, "tdc_pool2d_f32: mode %d", mode);
    if (2 * pad > window_h || 2 * pad > window_w)          // every window must hold at least one real element
        return fail(TDC_ERR_SHAPE, "tdc_pool2d_f32: padding %d leaves windows of %dx%d with no real element", pad, window_h, window_w);
    if (H + 2 * pad < window_h || W + 2 * pad < window_w)
        return fail(TDC_ERR_SHAPE, "tdc_pool2d_f32: window %dx%d larger than the padded %dx%d image", window_h, window_w, H, W);
    const int Ho = (H - window_h + 2 * pad) / stride + 1, Wo = (W - window_w + 2 * pad) / stride + 1;
    const long long planes = (long long)B * C;
    cudaStream_t st = (cudaStream_t)stream;
    const bool fast = mode == TDC_POOL_MAX && window_h == 3 && window_w == 3 && stride == 2 && pad == 1 && W % 8 == 0 &&
                      reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0;
    const bool fast2 = mode == TDC_POOL_MAX && window_h == 2 && window_w == 2 && stride == 2 && pad == 0 && W % 8 == 0 && H % 2 == 0 &&
                       reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0;
    const long long n = (fast || fast2) ? planes * Ho * (Wo / 4) : planes * Ho * Wo;
    const int threads = 256;
    long long blocks = (n + threads - 1) / threads;
    if (blocks > 148ll * 64) blocks = 148ll * 64;
    if (fast) maxpool_3x3s2_kernel<<<(unsigned)blocks, threads, 0, st>>>(x, y, planes, H, W, Ho, Wo);
    else if (fast2) maxpool_2x2s2_kernel<<<(unsigned)blocks, threads, 0, st>>>(x, y, planes, H, W, Ho, Wo);
    else pool_generic_kernel<<<(unsigned)blocks, threads, 0, st>>>(x, y, planes, H, W, Ho, Wo, window_h, window_w, pad, stride, mode);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? TDC_OK : fail(TDC_ERR_CUDA, "tdc_pool2d_f32 launch: %s", cudaGetErrorString(e));
}
