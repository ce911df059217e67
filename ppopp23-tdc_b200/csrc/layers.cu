// Layer objects with the surface of the reference's end-to-end classes
// (A100-evaluation/EndToEnd/resnet18-tk/inc/common.h:38-69,158-166; src/Conv.cu:2-125;
// src/BasicBlock.cu:15-32): a layer is created for one fixed shape, owns its weights and
// its output buffer, and forward() hands back that buffer.  The *_host calls wrap the
// same forward in the copy-in / run / copy-out sequence of the per-shape drivers' main()
// (A100-evaluation/TDC-LAYERS-ORACLE/template_benchmark_cudnn.template:412-498).
#include <cuda_runtime.h>
#include <algorithm>
#include <cstdio>
#include <vector>
#include "../../include/tdc_b200.h"
#include "errors.h"

struct tdc_conv {
    int b, c, h, w, n, pad, r, s, stride, ho, wo;
    float *kernel = nullptr, *bias = nullptr, *output = nullptr, *staging_in = nullptr;
    bool has_tile = false;
    tdc_tile tile{};
    int tc_mode = 0;            // 0: fp32 kernels; 1 / 3: tensor cores (TF32 / 3xTF32)
    tdc_tc_plan plan{};
    void* tc_weights = nullptr;
    float* kcrs = nullptr;      // the filter as given, kept for tdc_conv_set_precision
    cudaStream_t side[2] = {nullptr, nullptr};      // tdc_conv_forward_host_async: the chunks of a batch alternate between them
    cudaEvent_t side_done[2] = {nullptr, nullptr}, start = nullptr;
};

struct tdc_tkconv {
    int b, C, N1, N2, N3, h, w, r, s, pad, stride, ho, wo;
    float *w1 = nullptr, *wcore = nullptr, *w3 = nullptr, *bias = nullptr;
    float *output = nullptr, *staging_in = nullptr;
    void* workspace = nullptr;
    size_t workspace_bytes = 0;
    std::vector<float> h_w1, h_core, h_w3;   // the factors as given (all ones when none were), for tdc_tkconv_set_precision
    int tc_mode = 0;                         // 0: the three fp32 launches; 1 / 3 / 4: ONE tensor-core launch on the merged filter
    tdc_tc_plan plan{};
    void* tc_weights = nullptr;
};

namespace {

using tdc::fail;

int cuda_fail(const char* what, cudaError_t e) { return fail(TDC_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e)); }

int upload(float** dst, const float* host, size_t n, float fill_if_null) {
    cudaError_t e = cudaMalloc((void**)dst, n * sizeof(float));
    if (e != cudaSuccess) return cuda_fail("cudaMalloc", e);
    if (host) e = cudaMemcpy(*dst, host, n * sizeof(float), cudaMemcpyHostToDevice);
    else {
        std::vector<float> ones(n, fill_if_null);
        e = cudaMemcpy(*dst, ones.data(), n * sizeof(float), cudaMemcpyHostToDevice);
    }
    return e == cudaSuccess ? TDC_OK : cuda_fail("cudaMemcpy", e);
}

}  // namespace

extern "C" {

void tdc_conv_destroy(tdc_conv* l) {
    if (!l) return;
    cudaFree(l->kernel); cudaFree(l->bias); cudaFree(l->output); cudaFree(l->staging_in);
    cudaFree(l->tc_weights); cudaFree(l->kcrs);
    for (int i = 0; i < 2; ++i) {
        if (l->side[i]) cudaStreamDestroy(l->side[i]);
        if (l->side_done[i]) cudaEventDestroy(l->side_done[i]);
    }
    if (l->start) cudaEventDestroy(l->start);
    delete l;
}

int tdc_conv_set_precision(tdc_conv* l, int mode) {
    if (!l) return fail(TDC_ERR_NULL, "tdc_conv_set_precision: layer is NULL");
    if (mode == 0) { l->tc_mode = 0; return TDC_OK; }
    if (l->stride != 1 || l->r != l->s || (l->r != 1 && l->r != 3) || l->pad != (l->r - 1) / 2)
        return fail(TDC_ERR_UNSUPPORTED, "tdc_conv_set_precision: the tensor-core path of a layer object takes 1x1 and 3x3 filters, "
                                         "stride 1, padding (R-1)/2; this layer is %dx%d stride %d padding %d", l->r, l->s, l->stride, l->pad);
    tdc_tc_plan p;
    // the layer's shape is fixed, so the output-channel block size that suits its position count is known here
    tdc_devinfo dev;
    int rc = tdc_query_device(-1, &dev);
    if (rc) return rc;
    const int halo = (l->r - 1) / 2;
    int nt = tdc_tc_pick_nt(l->n, mode, (long long)l->b * (l->h + halo) * (l->w + halo), dev.sm_count);
    for (;; nt /= 2) {      // a wide image may not leave room for two stages beside a large block: take a smaller one
        rc = tdc_tc_plan_make_nt(l->c, l->n, l->r, l->s, mode, 0, nt, &p);
        if (rc) return rc;
        if (nt == 32 || tdc_tc_check_launch(&p, l->b, l->h, l->w, 0) != TDC_ERR_SMEM) break;
    }
    void* wt = nullptr;
    cudaError_t e = cudaMalloc(&wt, p.weights_bytes);
    if (e != cudaSuccess) return cuda_fail("cudaMalloc", e);
    rc = tdc_tc_prepare_weights(&p, l->kcrs, TDC_W_KCRS, wt, nullptr);
    e = cudaDeviceSynchronize();
    if (rc || e != cudaSuccess) { cudaFree(wt); return rc ? rc : cuda_fail("prepare", e); }
    cudaFree(l->tc_weights);
    l->tc_weights = wt; l->plan = p; l->tc_mode = mode;
    return TDC_OK;
}

int tdc_conv_create(tdc_conv** out, int b, int c, int h, int w, int n, int pad, int r, int s, int stride,
                    const float* host_w_kcrs, const float* host_bias) {
    if (!out) return fail(TDC_ERR_NULL, "tdc_conv_create: out is NULL");
    *out = nullptr;
    if (b <= 0 || c <= 0 || h <= 0 || w <= 0 || n <= 0 || r <= 0 || s <= 0 || stride <= 0 || pad < 0 ||
        h + 2 * pad < r || w + 2 * pad < s)
        return fail(TDC_ERR_SHAPE, "tdc_conv_create: b=%d c=%d h=%d w=%d n=%d filter %dx%d pad=%d stride=%d", b, c, h, w, n, r, s, pad, stride);
    tdc_conv* l = new tdc_conv;
    l->b = b; l->c = c; l->h = h; l->w = w; l->n = n; l->pad = pad; l->r = r; l->s = s; l->stride = stride;
    l->ho = (h + 2 * pad - r) / stride + 1;
    l->wo = (w + 2 * pad - s) / stride + 1;
    int rc;
    // Filter is kept channel-last ([c][r][s][n], the reference kernel's own layout) so the
    // kernel stages it with 16-byte copies.
    float* kcrs = nullptr;
    size_t wn = (size_t)n * c * r * s;
    if ((rc = upload(&kcrs, host_w_kcrs, wn, 1.0f))) { tdc_conv_destroy(l); return rc; }
    cudaError_t e = cudaMalloc((void**)&l->kernel, wn * sizeof(float));
    if (e != cudaSuccess) { cudaFree(kcrs); tdc_conv_destroy(l); return cuda_fail("cudaMalloc", e); }
    rc = tdc_permute_weights(kcrs, l->kernel, n, c, r, s, nullptr);
    e = cudaDeviceSynchronize();
    l->kcrs = kcrs;
    if (rc || e != cudaSuccess) { tdc_conv_destroy(l); return rc ? rc : cuda_fail("permute", e); }
    if (host_bias && (rc = upload(&l->bias, host_bias, n, 0.f))) { tdc_conv_destroy(l); return rc; }
    e = cudaMalloc((void**)&l->output, (size_t)b * n * l->ho * l->wo * sizeof(float));
    if (e != cudaSuccess) { tdc_conv_destroy(l); return cuda_fail("cudaMalloc", e); }
    *out = l;
    return TDC_OK;
}

int tdc_conv_set_tile(tdc_conv* l, const tdc_tile* tile) {
    if (!l) return fail(TDC_ERR_NULL, "tdc_conv_set_tile: layer is NULL");
    l->has_tile = tile != nullptr;
    if (tile) l->tile = *tile;
    return TDC_OK;
}

// Images [b0, b0 + nb) of the layer's batch: dev_in and the layer's output buffer are addressed at image b0.
static int conv_forward_images(tdc_conv* l, const float* dev_in, int b0, int nb, void* stream) {
    const float* x = dev_in + (size_t)b0 * l->c * l->h * l->w;
    float* y = l->output + (size_t)b0 * l->n * l->ho * l->wo;
    if (l->tc_mode) {
        tdc_epilogue e{nullptr, l->bias, nullptr, 0};
        // layer objects are chained into networks: sums without the tensor core's truncation bias
        return tdc_conv2d_tc(&l->plan, x, l->tc_weights, y, nb, l->h, l->w, &e, l->tc_mode == 1 ? 0 : TDC_TC_UNBIASED, stream);
    }
    return tdc_conv2d_f32(x, l->kernel, l->bias, y, nb, l->c, l->h, l->w, l->n, l->r, l->s, l->pad, l->stride, TDC_W_CRSK,
                          TDC_EPI_NONE, (l->has_tile && nb == l->b) ? &l->tile : nullptr, stream);
}

int tdc_conv_forward(tdc_conv* l, const float* dev_in, float** dev_out, void* stream) {
    if (!l || !dev_in || !dev_out) return fail(TDC_ERR_NULL, "tdc_conv_forward: layer, dev_in and dev_out must be non-NULL");
    int rc = conv_forward_images(l, dev_in, 0, l->b, stream);
    if (rc) return rc;
    *dev_out = l->output;
    return TDC_OK;
}

int tdc_conv_forward_host_async(tdc_conv* l, const float* host_in, float* host_out, void* stream) {
    if (!l || !host_in || !host_out) return fail(TDC_ERR_NULL, "tdc_conv_forward_host_async: layer, host_in and host_out must be non-NULL");
    const size_t in_img = (size_t)l->c * l->h * l->w, out_img = (size_t)l->n * l->ho * l->wo;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (!l->staging_in && (e = cudaMalloc((void**)&l->staging_in, l->b * in_img * sizeof(float))) != cudaSuccess) return cuda_fail("cudaMalloc", e);
    // A batch of several images goes through in chunks on two streams of the layer's own, so that the copy in of one
    // chunk, the kernel of another and the copy out of a third overlap; the caller's stream orders the whole
    // (work queued on it before this call precedes the first copy, work queued after it follows the last).
    const int chunks = (l->b >= 8 && l->b * (in_img + out_img) * sizeof(float) >= (4u << 20)) ? 4 : 1;
    if (chunks == 1) {
        if ((e = cudaMemcpyAsync(l->staging_in, host_in, l->b * in_img * sizeof(float), cudaMemcpyHostToDevice, st)) != cudaSuccess)
            return cuda_fail("copy in", e);
        int rc = conv_forward_images(l, l->staging_in, 0, l->b, stream);
        if (rc) return rc;
        e = cudaMemcpyAsync(host_out, l->output, l->b * out_img * sizeof(float), cudaMemcpyDeviceToHost, st);
        return e == cudaSuccess ? TDC_OK : cuda_fail("copy out", e);
    }
    if (!l->side[0]) {
        for (int i = 0; i < 2; ++i)
            if ((e = cudaStreamCreateWithFlags(&l->side[i], cudaStreamNonBlocking)) != cudaSuccess ||
                (e = cudaEventCreateWithFlags(&l->side_done[i], cudaEventDisableTiming)) != cudaSuccess)
                return cuda_fail("side stream", e);
        if ((e = cudaEventCreateWithFlags(&l->start, cudaEventDisableTiming)) != cudaSuccess) return cuda_fail("event", e);
    }
    if ((e = cudaEventRecord(l->start, st)) != cudaSuccess) return cuda_fail("event record", e);
    for (int i = 0; i < 2; ++i)
        if ((e = cudaStreamWaitEvent(l->side[i], l->start, 0)) != cudaSuccess) return cuda_fail("stream wait", e);
    for (int k = 0; k < chunks; ++k) {
        const int b0 = (int)((long long)l->b * k / chunks), nb = (int)((long long)l->b * (k + 1) / chunks) - b0;
        cudaStream_t s = l->side[k & 1];
        if ((e = cudaMemcpyAsync(l->staging_in + b0 * in_img, host_in + b0 * in_img, nb * in_img * sizeof(float), cudaMemcpyHostToDevice, s)) != cudaSuccess)
            return cuda_fail("copy in", e);
        int rc = conv_forward_images(l, l->staging_in, b0, nb, s);
        if (rc) return rc;
        if ((e = cudaMemcpyAsync(host_out + b0 * out_img, l->output + b0 * out_img, nb * out_img * sizeof(float), cudaMemcpyDeviceToHost, s)) != cudaSuccess)
            return cuda_fail("copy out", e);
    }
    for (int i = 0; i < 2; ++i)
        if ((e = cudaEventRecord(l->side_done[i], l->side[i])) != cudaSuccess || (e = cudaStreamWaitEvent(st, l->side_done[i], 0)) != cudaSuccess)
            return cuda_fail("join", e);
    return TDC_OK;
}

int tdc_conv_forward_host(tdc_conv* l, const float* host_in, float* host_out) {
    int rc = tdc_conv_forward_host_async(l, host_in, host_out, nullptr);
    if (rc) return rc;
    cudaError_t e = cudaStreamSynchronize(nullptr);
    return e == cudaSuccess ? TDC_OK : cuda_fail("synchronize", e);
}

void tdc_tkconv_destroy(tdc_tkconv* l) {
    if (!l) return;
    cudaFree(l->w1); cudaFree(l->wcore); cudaFree(l->w3); cudaFree(l->bias);
    cudaFree(l->output); cudaFree(l->staging_in); cudaFree(l->workspace); cudaFree(l->tc_weights);
    delete l;
}

int tdc_tkconv_create(tdc_tkconv** out, int b, int C, int N1, int N2, int N3, int h, int w, int r, int s, int pad,
                      int stride, const float* host_w1, const float* host_wcore_kcrs, const float* host_w3,
                      const float* host_bias) {
    if (!out) return fail(TDC_ERR_NULL, "tdc_tkconv_create: out is NULL");
    *out = nullptr;
    if (b <= 0 || C <= 0 || N1 <= 0 || N2 <= 0 || N3 <= 0 || h <= 0 || w <= 0 || r <= 0 || s <= 0 || stride <= 0 ||
        pad < 0 || h + 2 * pad < r || w + 2 * pad < s)
        return fail(TDC_ERR_SHAPE, "tdc_tkconv_create: b=%d C=%d N1=%d N2=%d N3=%d h=%d w=%d filter %dx%d pad=%d stride=%d", b, C, N1, N2,
                    N3, h, w, r, s, pad, stride);
    tdc_tkconv* l = new tdc_tkconv;
    l->b = b; l->C = C; l->N1 = N1; l->N2 = N2; l->N3 = N3; l->h = h; l->w = w; l->r = r; l->s = s;
    l->pad = pad; l->stride = stride;
    l->h_w1.assign((size_t)N1 * C, 1.0f); l->h_core.assign((size_t)N2 * N1 * r * s, 1.0f); l->h_w3.assign((size_t)N3 * N2, 1.0f);
    if (host_w1) l->h_w1.assign(host_w1, host_w1 + l->h_w1.size());
    if (host_wcore_kcrs) l->h_core.assign(host_wcore_kcrs, host_wcore_kcrs + l->h_core.size());
    if (host_w3) l->h_w3.assign(host_w3, host_w3 + l->h_w3.size());
    l->ho = (h + 2 * pad - r) / stride + 1;
    l->wo = (w + 2 * pad - s) / stride + 1;
    int rc;
    if ((rc = upload(&l->w1, host_w1, (size_t)N1 * C, 1.0f))) { tdc_tkconv_destroy(l); return rc; }
    if ((rc = upload(&l->w3, host_w3, (size_t)N3 * N2, 1.0f))) { tdc_tkconv_destroy(l); return rc; }
    float* kcrs = nullptr;
    size_t wn = (size_t)N2 * N1 * r * s;
    if ((rc = upload(&kcrs, host_wcore_kcrs, wn, 1.0f))) { tdc_tkconv_destroy(l); return rc; }
    cudaError_t e = cudaMalloc((void**)&l->wcore, wn * sizeof(float));
    if (e != cudaSuccess) { cudaFree(kcrs); tdc_tkconv_destroy(l); return cuda_fail("cudaMalloc", e); }
    rc = tdc_permute_weights(kcrs, l->wcore, N2, N1, r, s, nullptr);
    e = cudaDeviceSynchronize();
    cudaFree(kcrs);
    if (rc || e != cudaSuccess) { tdc_tkconv_destroy(l); return rc ? rc : cuda_fail("permute", e); }
    if (host_bias && (rc = upload(&l->bias, host_bias, N3, 0.f))) { tdc_tkconv_destroy(l); return rc; }
    l->workspace_bytes = tdc_tk_block_workspace_bytes(b, C, h, w, N1, N2, N3, r, s, pad, stride);
    if ((e = cudaMalloc(&l->workspace, l->workspace_bytes)) != cudaSuccess ||
        (e = cudaMalloc((void**)&l->output, (size_t)b * N3 * l->ho * l->wo * sizeof(float))) != cudaSuccess) {
        tdc_tkconv_destroy(l);
        return cuda_fail("cudaMalloc", e);
    }
    *out = l;
    return TDC_OK;
}

int tdc_tkconv_set_precision(tdc_tkconv* l, int mode) {
    if (!l) return fail(TDC_ERR_NULL, "tdc_tkconv_set_precision: layer is NULL");
    if (mode == 0) { l->tc_mode = 0; return TDC_OK; }
    if (l->r != l->s) return fail(TDC_ERR_UNSUPPORTED, "tdc_tkconv_set_precision: the merged form takes square filters, this layer is %dx%d", l->r, l->s);
    // w[k][c][i][j] = sum_{r2, r1} w3[k][r2] * core[r2][r1][i][j] * w1[r1][c], in double, rounded once: the weight the
    // reference's TKConv2dR recovers before its single conv (inference/TKConv.py:310-322)
    const int C = l->C, N1 = l->N1, N2 = l->N2, N3 = l->N3, rs = l->r * l->s;
    std::vector<double> t((size_t)N2 * C * rs, 0.0);                 // core x w1: [r2][c][ij]
    for (int r2 = 0; r2 < N2; ++r2)
        for (int r1 = 0; r1 < N1; ++r1)
            for (int ij = 0; ij < rs; ++ij) {
                const double cv = l->h_core[((size_t)r2 * N1 + r1) * rs + ij];
                double* trow = &t[(size_t)r2 * C * rs + ij];
                const float* w1row = &l->h_w1[(size_t)r1 * C];
                for (int c = 0; c < C; ++c) trow[(size_t)c * rs] += cv * w1row[c];
            }
    std::vector<float> merged((size_t)N3 * C * rs);
    std::vector<double> acc((size_t)C * rs);
    for (int k = 0; k < N3; ++k) {
        std::fill(acc.begin(), acc.end(), 0.0);
        for (int r2 = 0; r2 < N2; ++r2) {
            const double wv = l->h_w3[(size_t)k * N2 + r2];
            const double* trow = &t[(size_t)r2 * C * rs];
            for (size_t i = 0; i < acc.size(); ++i) acc[i] += wv * trow[i];
        }
        for (size_t i = 0; i < acc.size(); ++i) merged[(size_t)k * C * rs + i] = (float)acc[i];
    }
    const bool one_pass = l->stride == 1 && l->pad == (l->r - 1) / 2 && (l->r == 1 || l->r == 3);
    tdc_tc_plan p;
    tdc_devinfo dev;
    int rc = tdc_query_device(-1, &dev);
    if (rc) return rc;
    const int halo = one_pass ? (l->r - 1) / 2 : 0;
    const int flags = (l->stride - 1) | (one_pass ? 0 : (l->pad << TDC_TC_PAD_SHIFT));
    int nt = tdc_tc_pick_nt(N3, mode, (long long)l->b * (l->ho + halo) * (l->wo + halo), dev.sm_count);
    for (;; nt /= 2) {      // the block size that suits the layer's position count and still fits beside a wide image's patch
        rc = tdc_tc_plan_make_nt(C, N3, l->r, l->s, mode, one_pass ? 0 : 1, nt, &p);
        if (rc) return rc;
        if (nt == 32 || tdc_tc_check_launch(&p, l->b, l->h, l->w, flags) != TDC_ERR_SMEM) break;
    }
    float* dev_w = nullptr;
    void* wt = nullptr;
    cudaError_t e;
    if ((e = cudaMalloc((void**)&dev_w, merged.size() * sizeof(float))) != cudaSuccess || (e = cudaMalloc(&wt, p.weights_bytes)) != cudaSuccess) {
        cudaFree(dev_w);
        return cuda_fail("cudaMalloc", e);
    }
    e = cudaMemcpy(dev_w, merged.data(), merged.size() * sizeof(float), cudaMemcpyHostToDevice);
    rc = e == cudaSuccess ? tdc_tc_prepare_weights(&p, dev_w, TDC_W_KCRS, wt, nullptr) : cuda_fail("cudaMemcpy", e);
    if (!rc && (e = cudaDeviceSynchronize()) != cudaSuccess) rc = cuda_fail("prepare", e);
    cudaFree(dev_w);
    if (rc) { cudaFree(wt); return rc; }
    cudaFree(l->tc_weights);
    l->tc_weights = wt; l->plan = p; l->tc_mode = mode;
    return TDC_OK;
}

int tdc_tkconv_forward(tdc_tkconv* l, const float* dev_in, float** dev_out, void* stream) {
    if (!l || !dev_in || !dev_out) return fail(TDC_ERR_NULL, "tdc_tkconv_forward: layer, dev_in and dev_out must be non-NULL");
    if (l->tc_mode) {
        tdc_epilogue e{nullptr, l->bias, nullptr, 0};
        const int flags = (l->stride - 1) | (l->plan.general ? (l->pad << TDC_TC_PAD_SHIFT) : 0) | (l->tc_mode == 1 ? 0 : TDC_TC_UNBIASED);
        const int rc = tdc_conv2d_tc(&l->plan, dev_in, l->tc_weights, l->output, l->b, l->h, l->w, &e, flags, stream);
        if (rc) return rc;
        *dev_out = l->output;
        return TDC_OK;
    }
    int rc = tdc_tk_block_f32(dev_in, l->w1, l->wcore, l->w3, l->bias, l->output, l->b, l->C, l->h, l->w, l->N1,
                              l->N2, l->N3, l->r, l->s, l->pad, l->stride, TDC_W_CRSK, TDC_EPI_NONE, nullptr, l->workspace,
                              l->workspace_bytes, stream);
    if (rc) return rc;
    *dev_out = l->output;
    return TDC_OK;
}

int tdc_tkconv_forward_host(tdc_tkconv* l, const float* host_in, float* host_out) {
    if (!l || !host_in || !host_out) return fail(TDC_ERR_NULL, "tdc_tkconv_forward_host: layer, host_in and host_out must be non-NULL");
    size_t in_bytes = (size_t)l->b * l->C * l->h * l->w * sizeof(float);
    cudaError_t e;
    if (!l->staging_in && (e = cudaMalloc((void**)&l->staging_in, in_bytes)) != cudaSuccess) return cuda_fail("cudaMalloc", e);
    if ((e = cudaMemcpyAsync(l->staging_in, host_in, in_bytes, cudaMemcpyHostToDevice, nullptr)) != cudaSuccess)
        return cuda_fail("copy in", e);
    float* o;
    int rc = tdc_tkconv_forward(l, l->staging_in, &o, nullptr);
    if (rc) return rc;
    e = cudaMemcpyAsync(host_out, o, (size_t)l->b * l->N3 * l->ho * l->wo * sizeof(float), cudaMemcpyDeviceToHost, nullptr);
    if (e != cudaSuccess) return cuda_fail("copy out", e);
    e = cudaStreamSynchronize(nullptr);
    return e == cudaSuccess ? TDC_OK : cuda_fail("synchronize", e);
}

}  // extern "C"
