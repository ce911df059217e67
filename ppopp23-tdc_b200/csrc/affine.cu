// Per-channel scale, shift and ReLU with image strides: the pre-activation layers of the DenseNet skeleton.  One
// launch stands for the reference's BatchNorm::forward (inference form, y = x*scale + shift once mean and variance
// are folded in; A100-evaluation/EndToEnd/densenet121-tk/src/BatchNorm.cu:58-80) followed by Activation::forward
// (src/Activation.cu:38-41), and — with a destination stride larger than C*HW and no scale — for the copy of a
// layer's new features into the block's concatenated feature buffer (Concate::forward, inc/common.h:165-177;
// TenDenseLayer::forward, src/TenDense.cu:44-53; torch.cat in inference/densenet_inet_tt.py:58-60,134-139).
// Memory-bound: every element read once, written once.
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/tdc_b200.h"
#include "errors.h"

namespace {

// One thread per 16-byte group (V = 4) or per element (V = 1), grid-stride over all planes; IDX is 32-bit when the
// tensor allows it (the index arithmetic is then a handful of instructions beside the 16-byte access).
template <int V, typename IDX>
__global__ void __launch_bounds__(256) affine_relu_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                          const float* __restrict__ scale, const float* __restrict__ shift, int C,
                                                          int per, long long x_stride, long long y_stride, IDX total, int relu) {
    const IDX step = (IDX)gridDim.x * blockDim.x;
    for (IDX i = (IDX)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
        const IDX p = i / (IDX)per;                 // plane = image * C + channel
        const int r = (int)(i - p * (IDX)per);
        const IDX b = p / (IDX)C;
        const int c = (int)(p - b * (IDX)C);
        const float s = scale ? __ldg(scale + c) : 1.f, t = shift ? __ldg(shift + c) : 0.f;
        const long long off = (long long)c * per * V + (long long)r * V;
        const float* xp = x + (long long)b * x_stride + off;
        float* yp = y + (long long)b * y_stride + off;
        if (V == 4) {
            float4 v = __ldg(reinterpret_cast<const float4*>(xp));
            v.x = fmaf(v.x, s, t); v.y = fmaf(v.y, s, t); v.z = fmaf(v.z, s, t); v.w = fmaf(v.w, s, t);
            if (relu) { v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f); }
            *reinterpret_cast<float4*>(yp) = v;
        } else {
            const float v = fmaf(__ldg(xp), s, t);
            *yp = relu ? fmaxf(v, 0.f) : v;
        }
    }
}

template <int V>
void launch_affine(const float* x, float* y, const float* scale, const float* shift, int C, int per, long long xs, long long ys,
                   long long total, int relu, cudaStream_t st) {
    const int threads = 256;
    long long blocks = (total + threads - 1) / threads;
    if (blocks > 148ll * 32) blocks = 148ll * 32;
    if (total < (1ll << 31))
        affine_relu_kernel<V, unsigned><<<(unsigned)blocks, threads, 0, st>>>(x, y, scale, shift, C, per, xs, ys, (unsigned)total, relu);
    else
        affine_relu_kernel<V, long long><<<(unsigned)blocks, threads, 0, st>>>(x, y, scale, shift, C, per, xs, ys, total, relu);
}

}  // namespace

extern "C" int tdc_affine_relu_f32(const float* x, float* y, const float* scale, const float* shift, int B, int C, int HW,
                                   long long x_image_stride, long long y_image_stride, int relu, void* stream) {
    using tdc::fail;
    if (!x || !y) return fail(TDC_ERR_NULL, "tdc_affine_relu_f32: x and y must be non-NULL");
    if (B <= 0 || C <= 0 || HW <= 0) return fail(TDC_ERR_SHAPE, "tdc_affine_relu_f32: B=%d C=%d HW=%d", B, C, HW);
    if (x_image_stride < (long long)C * HW || y_image_stride < (long long)C * HW)
        return fail(TDC_ERR_SHAPE, "tdc_affine_relu_f32: image strides %lld / %lld are shorter than an image of %lld elements",
                    x_image_stride, y_image_stride, (long long)C * HW);
    const long long planes = (long long)B * C;
    const bool vec = HW % 4 == 0 && x_image_stride % 4 == 0 && y_image_stride % 4 == 0 &&
                     reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (vec) launch_affine<4>(x, y, scale, shift, C, HW / 4, x_image_stride, y_image_stride, planes * (HW / 4), relu, st);
    else launch_affine<1>(x, y, scale, shift, C, HW, x_image_stride, y_image_stride, planes * HW, relu, st);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? TDC_OK : fail(TDC_ERR_CUDA, "tdc_affine_relu_f32 launch: %s", cudaGetErrorString(e));
}
