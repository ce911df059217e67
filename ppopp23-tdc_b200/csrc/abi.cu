// The extern "C" surface of libtdc_b200.so (declared in include/tdc_b200.h): argument
// checks, tile completion, launches, the weight permutation and the three-step Tucker
// block.  Nothing here exits the process or throws across the boundary; the reference
// drivers' error path is exit(-1)
// (A100-evaluation/TDC-LAYERS-ORACLE/template_benchmark_cudnn.template:31-47).
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>
#include "errors.h"
#include "tile.h"

namespace tdc {
static thread_local char g_err[512] = "";
int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return code;
}
const char* last_error() { return g_err; }
}  // namespace tdc

using namespace tdc;

namespace {

#ifdef TDC_DEBUG_BOUNDS
__device__ int g_debug_bounds[4];     // see ConvArgs::bounds
#endif
std::mutex g_mu;
std::map<int, tdc_devinfo> g_dev;                          // per device
std::map<std::pair<int, const void*>, size_t> g_smem_set;  // (device, kernel) -> opted-in bytes
using ShapeKey = std::tuple<int, int, int, int, int, int, int, int, int, int>;
std::map<ShapeKey, tdc_tile> g_auto_tiles;                 // (device, shape) -> selected tile

int current_device(int* dev) {
    cudaError_t e = cudaGetDevice(dev);
    if (e != cudaSuccess) return fail(TDC_ERR_NO_DEVICE, "cudaGetDevice: %s", cudaGetErrorString(e));
    return TDC_OK;
}

int devinfo(int device, tdc_devinfo* out) {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_dev.find(device);
    if (it != g_dev.end()) { *out = it->second; return TDC_OK; }
    tdc_devinfo d;
    cudaError_t e;
    if ((e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&d.smem_per_cta, cudaDevAttrMaxSharedMemoryPerBlockOptin, device)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&d.regs_per_sm, cudaDevAttrMaxRegistersPerMultiprocessor, device)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&d.threads_per_sm, cudaDevAttrMaxThreadsPerMultiProcessor, device)) != cudaSuccess)
        return fail(TDC_ERR_NO_DEVICE, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
    g_dev[device] = d;
    *out = d;
    return TDC_OK;
}

int check_shape(const Shape& s) {
    if (s.B <= 0 || s.C <= 0 || s.H <= 0 || s.W <= 0 || s.K <= 0 || s.R <= 0 || s.S <= 0)
        return fail(TDC_ERR_SHAPE, "non-positive dimension (B=%d C=%d H=%d W=%d K=%d R=%d S=%d)", s.B, s.C, s.H,
                    s.W, s.K, s.R, s.S);
    if (s.pad < 0 || s.stride <= 0) return fail(TDC_ERR_SHAPE, "pad=%d stride=%d", s.pad, s.stride);
    if (s.H + 2 * s.pad < s.R || s.W + 2 * s.pad < s.S)
        return fail(TDC_ERR_SHAPE, "filter %dx%d larger than padded input %dx%d", s.R, s.S, s.H + 2 * s.pad,
                    s.W + 2 * s.pad);
    if (s.stride > 2) return fail(TDC_ERR_UNSUPPORTED, "stride %d (1 and 2 are built)", s.stride);
    if (s.R > 7 || s.S > 7) return fail(TDC_ERR_UNSUPPORTED, "filter %dx%d (up to 7x7 is built)", s.R, s.S);
    return TDC_OK;
}

bool tile_complete(const tdc_tile& t) {
    return t.th && t.tw && t.tc && t.tn && t.nog && t.gy && t.gx && t.imgs && t.ks && t.kc;
}

// Completes *t (zero fields) for the shape on `dev`; caches fully automatic choices.
int complete_tile(const Shape& s, int device, const tdc_devinfo& dev, tdc_tile* t) {
    if (tile_complete(*t)) return TDC_OK;
    const bool all_auto = !t->th && !t->tw && !t->tc && !t->tn && !t->nog && !t->gy && !t->gx && !t->imgs && !t->ks && !t->kc;
    ShapeKey key{device, s.B, s.C, s.H, s.W, s.K, s.R, s.S, s.pad, s.stride};
    if (all_auto && device >= 0) {
        std::lock_guard<std::mutex> lk(g_mu);
        auto it = g_auto_tiles.find(key);
        if (it != g_auto_tiles.end()) { *t = it->second; return TDC_OK; }
    }
    tdc_tile out;
    int rc = select_tile(s, dev, *t, &out);
    if (rc != TDC_OK) return fail(rc, "no tile fits this shape with the fields given");
    *t = out;
    if (all_auto && device >= 0) {
        std::lock_guard<std::mutex> lk(g_mu);
        g_auto_tiles[key] = out;
    }
    return TDC_OK;
}

int launch_conv_epi(const float* x, const float* w, const tdc_epilogue& epi, float* y, const Shape& s, int w_layout,
                    const tdc_tile* tile_in, cudaStream_t stream);

int launch_conv(const float* x, const float* w, const float* bias, float* y, const Shape& s, int w_layout,
                int epilogue, const tdc_tile* tile_in, cudaStream_t stream) {
    tdc_epilogue epi{nullptr, bias, nullptr, (epilogue & TDC_EPI_RELU) ? 1 : 0};
    return launch_conv_epi(x, w, epi, y, s, w_layout, tile_in, stream);
}

int launch_conv_epi(const float* x, const float* w, const tdc_epilogue& epi, float* y, const Shape& s, int w_layout,
                    const tdc_tile* tile_in, cudaStream_t stream) {
    if (!x || !w || !y) return fail(TDC_ERR_NULL, "x, w and y must be non-NULL");
    int rc = check_shape(s);
    if (rc) return rc;
    if (w_layout != TDC_W_KCRS && w_layout != TDC_W_CRSK) return fail(TDC_ERR_UNSUPPORTED, "w_layout %d", w_layout);
    int device;
    if ((rc = current_device(&device))) return rc;
    tdc_devinfo dev;
    if ((rc = devinfo(device, &dev))) return rc;
    tdc_tile t{};
    if (tile_in) t = *tile_in;
    if ((rc = complete_tile(s, device, dev, &t))) return rc;
    Geometry g;
    const char* why = "";
    if ((rc = make_geometry(s, t, dev, &g, &why))) return fail(rc, "%s", why);

    ConvArgs a;
    a.x = x; a.w = w; a.bias = epi.bias; a.scale = epi.scale; a.residual = epi.residual; a.y = y;
    a.B = s.B; a.C = s.C; a.H = s.H; a.W = s.W; a.K = s.K; a.Ho = s.Ho(); a.Wo = s.Wo(); a.pad = s.pad;
    a.R = s.R; a.S = s.S;
    const int RS = s.R * s.S;
    if (w_layout == TDC_W_KCRS) { a.ws_k = (long long)s.C * RS; a.ws_c = RS; a.ws_rs = 1; }
    else                        { a.ws_k = 1; a.ws_c = (long long)RS * s.K; a.ws_rs = s.K; }
    a.w_vec = (w_layout == TDC_W_CRSK && s.K % 4 == 0 && (reinterpret_cast<uintptr_t>(w) % 16 == 0)) ? 1 : 0;
    a.y_vec = reinterpret_cast<uintptr_t>(y) % 16 == 0 ? 1 : 0;      // else the epilogue stores element by element
    a.x_n = (long long)s.B * s.C * s.H * s.W; a.w_n = (long long)s.K * s.C * RS; a.y_n = (long long)s.B * s.K * s.Ho() * s.Wo();
    a.bounds = nullptr;
#ifdef TDC_DEBUG_BOUNDS
    {
        void* bp = nullptr;
        if (cudaGetSymbolAddress(&bp, g_debug_bounds) == cudaSuccess) a.bounds = (int*)bp;
    }
#endif
    a.relu = epi.relu ? 1 : 0;
    a.tc = t.tc; a.gy = t.gy; a.gx = t.gx; a.imgs = t.imgs; a.ks = t.ks;
    a.in_rows = g.in_rows; a.in_wp = g.in_wp; a.patch = g.patch;
    a.tiles_y = g.tiles_y; a.tiles_x = g.tiles_x; a.img_groups = g.img_groups; a.n_ocb = g.n_ocb;
    a.stage_floats = g.stage_floats;
    a.kc = t.kc; a.chunks_per_rank = g.chunks_per_rank;

    {
        std::lock_guard<std::mutex> lk(g_mu);
        size_t& have = g_smem_set[{device, g.v->fn}];
        if (g.smem_bytes > have) {
            cudaError_t e = cudaFuncSetAttribute(g.v->fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem_bytes);
            if (e != cudaSuccess) return fail(TDC_ERR_CUDA, "cudaFuncSetAttribute(%zu B): %s", g.smem_bytes, cudaGetErrorString(e));
            have = g.smem_bytes;
        }
    }
    void* args[] = {&a};
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)g.ctas);
    cfg.blockDim = dim3(g.threads);
    cfg.dynamicSmemBytes = g.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (t.kc > 1) {   // the kc CTAs of a tile form one thread-block cluster
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = t.kc; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
    }
    cudaError_t e = cudaLaunchKernelExC(&cfg, g.v->fn, args);
    if (e != cudaSuccess) return fail(TDC_ERR_CUDA, "launch: %s", cudaGetErrorString(e));
    return TDC_OK;
}

__global__ void permute_kcrs_to_crsk(const float* __restrict__ in, float* __restrict__ out, int K, int C, int RS) {
    // out[(c*RS + rs)*K + k] = in[(k*C + c)*RS + rs]; consecutive threads write consecutive k.
    long long n = (long long)K * C * RS;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        int k = (int)(i % K);
        long long q = i / K;   // c*RS + rs
        out[i] = in[(long long)k * C * RS + q];
    }
}

}  // namespace

extern "C" {

const char* tdc_last_error_string(void) { return tdc::last_error(); }
int tdc_version(void) { return 100; }

#ifdef TDC_DEBUG_BOUNDS
// Range-checked build only: {violations, kind of the first, its offset (low, high word)} of all fp32-kernel launches so
// far on the current device; reset != 0 clears the record.  Synchronises.
__attribute__((visibility("default"))) int tdc_debug_bounds_read(int* out4, int reset) {
    cudaError_t e = cudaMemcpyFromSymbol(out4, g_debug_bounds, 4 * sizeof(int));
    if (e == cudaSuccess && reset) { const int z[4] = {0, 0, 0, 0}; e = cudaMemcpyToSymbol(g_debug_bounds, z, sizeof z); }
    return e == cudaSuccess ? TDC_OK : fail(TDC_ERR_CUDA, "bounds record: %s", cudaGetErrorString(e));
}
#endif

int tdc_query_device(int device, tdc_devinfo* out) {
    if (!out) return fail(TDC_ERR_NULL, "out is NULL");
    int rc;
    if (device < 0 && (rc = current_device(&device))) return rc;
    return devinfo(device, out);
}

int tdc_core_conv2d_f32(const float* x, const float* w, float* y, int B, int C, int H, int W, int K, int R, int S,
                        int pad, int stride, int w_layout, const tdc_tile* tile, void* stream) {
    return launch_conv(x, w, nullptr, y, Shape{B, C, H, W, K, R, S, pad, stride}, w_layout, TDC_EPI_NONE, tile,
                       (cudaStream_t)stream);
}

int tdc_conv2d_f32(const float* x, const float* w, const float* bias, float* y, int B, int C, int H, int W, int K,
                   int R, int S, int pad, int stride, int w_layout, int epilogue, const tdc_tile* tile, void* stream) {
    return launch_conv(x, w, bias, y, Shape{B, C, H, W, K, R, S, pad, stride}, w_layout, epilogue, tile,
                       (cudaStream_t)stream);
}

int tdc_conv2d_epi_f32(const float* x, const float* w, float* y, int B, int C, int H, int W, int K, int R, int S,
                       int pad, int stride, int w_layout, const tdc_epilogue* epi, const tdc_tile* tile, void* stream) {
    tdc_epilogue e{nullptr, nullptr, nullptr, 0};
    if (epi) e = *epi;
    return launch_conv_epi(x, w, e, y, Shape{B, C, H, W, K, R, S, pad, stride}, w_layout, tile, (cudaStream_t)stream);
}

int tdc_permute_weights(const float* w_kcrs, float* w_crsk, int K, int C, int R, int S, void* stream) {
    if (!w_kcrs || !w_crsk) return fail(TDC_ERR_NULL, "weights pointer is NULL");
    if (K <= 0 || C <= 0 || R <= 0 || S <= 0) return fail(TDC_ERR_SHAPE, "non-positive filter dimension");
    long long n = (long long)K * C * R * S;
    int blocks = (int)std::min<long long>((n + 255) / 256, 148 * 8);
    permute_kcrs_to_crsk<<<blocks, 256, 0, (cudaStream_t)stream>>>(w_kcrs, w_crsk, K, C, R * S);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(TDC_ERR_CUDA, "permute launch: %s", cudaGetErrorString(e));
    return TDC_OK;
}

static int dev_or_query(const tdc_devinfo* dev, tdc_devinfo* out, int* device) {
    *device = -1;
    if (dev) { *out = *dev; return TDC_OK; }
    int rc;
    if ((rc = current_device(device))) return rc;
    return devinfo(*device, out);
}

int tdc_select_tile(int B, int C, int H, int W, int K, int R, int S, int pad, int stride, const tdc_devinfo* dev,
                    tdc_tile* out) {
    if (!out) return fail(TDC_ERR_NULL, "out is NULL");
    Shape s{B, C, H, W, K, R, S, pad, stride};
    int rc = check_shape(s);
    if (rc) return rc;
    tdc_devinfo d;
    int device;
    if ((rc = dev_or_query(dev, &d, &device))) return rc;
    tdc_tile t{};
    if ((rc = select_tile(s, d, t, out))) return fail(rc, "no tile fits this shape");
    return TDC_OK;
}

int tdc_tile_info(int B, int C, int H, int W, int K, int R, int S, int pad, int stride, tdc_tile* tile,
                  tdc_launch_info* info) {
    if (!tile || !info) return fail(TDC_ERR_NULL, "tile or info is NULL");
    Shape s{B, C, H, W, K, R, S, pad, stride};
    int rc = check_shape(s);
    if (rc) return rc;
    int device;
    if ((rc = current_device(&device))) return rc;
    tdc_devinfo dev;
    if ((rc = devinfo(device, &dev))) return rc;
    if ((rc = complete_tile(s, -1, dev, tile))) return rc;
    Geometry g;
    const char* why = "";
    if ((rc = make_geometry(s, *tile, dev, &g, &why))) return fail(rc, "%s", why);
    info->grid_x = (int)g.ctas; info->grid_y = 1; info->threads = g.threads; info->smem_bytes = g.smem_bytes;
    cudaFuncAttributes fa;
    cudaError_t e = cudaFuncGetAttributes(&fa, g.v->fn);
    if (e != cudaSuccess) return fail(TDC_ERR_CUDA, "cudaFuncGetAttributes: %s", cudaGetErrorString(e));
    info->regs_per_thread = fa.numRegs;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        size_t& have = g_smem_set[{device, g.v->fn}];
        if (g.smem_bytes > have) {
            e = cudaFuncSetAttribute(g.v->fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem_bytes);
            if (e != cudaSuccess) return fail(TDC_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
            have = g.smem_bytes;
        }
    }
    int nb = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, g.v->fn, g.threads, g.smem_bytes);
    if (e != cudaSuccess) return fail(TDC_ERR_CUDA, "occupancy query: %s", cudaGetErrorString(e));
    info->ctas_per_sm = nb;
    return TDC_OK;
}

int tdc_tile_cost(int B, int C, int H, int W, int K, int R, int S, int pad, int stride, const tdc_tile* tile,
                  const tdc_devinfo* dev, double* cost, double* vols) {
    if (!tile || !cost) return fail(TDC_ERR_NULL, "tile or cost is NULL");
    Shape s{B, C, H, W, K, R, S, pad, stride};
    int rc = check_shape(s);
    if (rc) return rc;
    tdc_devinfo d;
    int device;
    if ((rc = dev_or_query(dev, &d, &device))) return rc;
    Geometry g;
    const char* why = "";
    if ((rc = make_geometry(s, *tile, d, &g, &why))) return fail(rc, "%s", why);
    *cost = tile_cost(s, *tile, g, d, vols);
    return TDC_OK;
}

size_t tdc_tk_block_workspace_bytes(int B, int C, int H, int W, int R1, int R2, int K, int R, int S, int pad,
                                    int stride) {
    (void)C; (void)K;
    if (B <= 0 || H <= 0 || W <= 0 || R1 <= 0 || R2 <= 0 || stride <= 0) return 0;
    long long Ho = (H + 2 * pad - R) / stride + 1, Wo = (W + 2 * pad - S) / stride + 1;
    if (Ho <= 0 || Wo <= 0) return 0;
    size_t z1 = (size_t)B * R1 * H * W, z2 = (size_t)B * R2 * Ho * Wo;
    return 4 * (((z1 + 63) / 64) * 64 + z2);
}

int tdc_tk_block_epi_f32(const float* x, const float* w1, const float* wcore, const float* w3, float* y, int B, int C,
                         int H, int W, int R1, int R2, int K, int R, int S, int pad, int stride, int w_layout,
                         const tdc_epilogue* epi, const tdc_tile* core_tile, void* workspace, size_t workspace_bytes,
                         void* stream) {
    if (!x || !w1 || !wcore || !w3 || !y) return fail(TDC_ERR_NULL, "x, w1, wcore, w3 and y must be non-NULL");
    size_t need = tdc_tk_block_workspace_bytes(B, C, H, W, R1, R2, K, R, S, pad, stride);
    if (need == 0) return fail(TDC_ERR_SHAPE, "bad Tucker block shape");
    if (!workspace || workspace_bytes < need)
        return fail(TDC_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", need, workspace ? workspace_bytes : 0);
    const int Ho = (H + 2 * pad - R) / stride + 1, Wo = (W + 2 * pad - S) / stride + 1;
    float* z1 = (float*)workspace;
    float* z2 = z1 + (((size_t)B * R1 * H * W + 63) / 64) * 64;
    cudaStream_t st = (cudaStream_t)stream;
    tdc_epilogue e{nullptr, nullptr, nullptr, 0};
    if (epi) e = *epi;
    int rc;
    // 1x1 convs take their filter as [out][in] = KCRS with R=S=1.
    if ((rc = launch_conv(x, w1, nullptr, z1, Shape{B, C, H, W, R1, 1, 1, 0, 1}, TDC_W_KCRS, TDC_EPI_NONE, nullptr, st))) return rc;
    if ((rc = launch_conv(z1, wcore, nullptr, z2, Shape{B, R1, H, W, R2, R, S, pad, stride}, w_layout, TDC_EPI_NONE, core_tile, st))) return rc;
    return launch_conv_epi(z2, w3, e, y, Shape{B, R2, Ho, Wo, K, 1, 1, 0, 1}, TDC_W_KCRS, nullptr, st);
}

int tdc_tk_block_f32(const float* x, const float* w1, const float* wcore, const float* w3, const float* bias,
                     float* y, int B, int C, int H, int W, int R1, int R2, int K, int R, int S, int pad, int stride,
                     int w_layout, int epilogue, const tdc_tile* core_tile, void* workspace, size_t workspace_bytes,
                     void* stream) {
    tdc_epilogue e{nullptr, bias, nullptr, (epilogue & TDC_EPI_RELU) ? 1 : 0};
    return tdc_tk_block_epi_f32(x, w1, wcore, w3, y, B, C, H, W, R1, R2, K, R, S, pad, stride, w_layout, &e, core_tile,
                                workspace, workspace_bytes, stream);
}

}  // extern "C"

// ---- the no-allocation variant of the Tucker block ---------------------------------------
// The intermediates live in this array, which is part of the library image: a GPU holds it
// from library load to process exit.  Its name is only a handle in host code; the device
// address the kernels need comes from cudaGetSymbolAddress, looked up once per device.
static __device__ __align__(256) unsigned char g_static_workspace[TDC_STATIC_WORKSPACE_BYTES];

namespace {
std::map<int, void*> g_static_ws_ptr;   // device -> address of g_static_workspace there

int static_workspace(void** out) {
    int device, rc;
    if ((rc = current_device(&device))) return rc;
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_static_ws_ptr.find(device);
    if (it == g_static_ws_ptr.end()) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_workspace);   // current device == `device`
        if (e != cudaSuccess || !p)
            return fail(TDC_ERR_CUDA, "cudaGetSymbolAddress(static workspace): %s", cudaGetErrorString(e));
        it = g_static_ws_ptr.emplace(device, p).first;
    }
    *out = it->second;
    return TDC_OK;
}
}  // namespace

extern "C" int tdc_tk_block_f32_static(const float* x, const float* w1, const float* wcore, const float* w3,
                                       const float* bias, float* y, int B, int C, int H, int W, int R1, int R2,
                                       int K, int R, int S, int pad, int stride, int w_layout, int epilogue,
                                       const tdc_tile* core_tile, void* stream) {
    size_t need = tdc_tk_block_workspace_bytes(B, C, H, W, R1, R2, K, R, S, pad, stride);
    if (need == 0) return fail(TDC_ERR_SHAPE, "bad Tucker block shape");
    if (need > (size_t)TDC_STATIC_WORKSPACE_BYTES)
        return fail(TDC_ERR_WORKSPACE,
                    "this Tucker block needs %zu bytes for its intermediates, the built-in workspace holds %zu; "
                    "use tdc_tk_block_f32 with a caller-provided workspace",
                    need, (size_t)TDC_STATIC_WORKSPACE_BYTES);
    void* ws = nullptr;
    int rc = static_workspace(&ws);
    if (rc) return rc;
    return tdc_tk_block_f32(x, w1, wcore, w3, bias, y, B, C, H, W, R1, R2, K, R, S, pad, stride, w_layout, epilogue,
                            core_tile, ws, (size_t)TDC_STATIC_WORKSPACE_BYTES, stream);
}
