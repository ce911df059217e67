/*
 * tdc_b200.h — C ABI of libtdc_b200.so: the core convolution of a Tucker-factorised
 * conv layer (and the 1x1 convs around it) as hand-written sm_100a CUDA.
 *
 * Every entry point is extern "C", takes plain pointers and sizes, never throws and
 * never exits the process: it returns a tdc_status and leaves a message readable with
 * tdc_last_error_string() (thread-local).  All device work is asynchronous on the
 * stream the caller passes (a cudaStream_t cast to void*; NULL = the default stream).
 * Unless a comment says otherwise, pointers are DEVICE pointers to contiguous fp32
 * arrays that the caller owns.
 *
 * Alignment.  x, w, y and the epilogue arrays need only the 4-byte alignment of a float:
 * where a kernel would use 16-byte accesses it checks the pointer first and takes an
 * element-wise path otherwise (slower, same results).  Two exceptions, both buffers the
 * caller allocates for the library: the prepared filter of the tensor-core path (wt) must
 * be 16-byte aligned, or tdc_tc_prepare_weights / tdc_conv2d_tc return
 * TDC_ERR_UNSUPPORTED; tdc_pool2d_f32 and tdc_affine_relu_f32 likewise fall back to scalar
 * accesses for unaligned x / y.
 *
 * Naming.  The reference's CUDA drivers call the core conv's input channels C and its
 * output channels N, and hard-wire batch 1.  Here:  B = batch, C = input channels (R1
 * of the Tucker block), K = output channels (R2), H,W = input height/width, R,S =
 * filter height/width.  Output size: Ho = (H + 2*pad - R)/stride + 1, same for Wo.
 *
 * Each declaration cites the reference interface it stands in for, as
 * path-in-reference:line.
 */
#ifndef TDC_B200_H
#define TDC_B200_H

#include <stddef.h>

#if defined(__GNUC__)
#define TDC_API __attribute__((visibility("default")))
#else
#define TDC_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum tdc_status {
    TDC_OK              = 0,
    TDC_ERR_NULL        = 1, /* a required pointer is NULL                          */
    TDC_ERR_SHAPE       = 2, /* a dimension is <= 0, or the output would be empty   */
    TDC_ERR_UNSUPPORTED = 3, /* filter size / stride / layout this build lacks      */
    TDC_ERR_TILE        = 4, /* the tile does not fit the shape or the device       */
    TDC_ERR_SMEM        = 5, /* the tile needs more shared memory than a CTA has    */
    TDC_ERR_CUDA        = 6, /* a CUDA runtime call failed (message has the reason) */
    TDC_ERR_WORKSPACE   = 7, /* workspace missing or too small                      */
    TDC_ERR_NO_DEVICE   = 8  /* no CUDA device / driver                             */
} tdc_status;

/* Filter memory layouts. KCRS is torch's core_kernel[R2][R1][kh][kw]
 * (inference/TKConv.py:63); CRSK is the reference CUDA kernel's k[c][r][s][n]
 * (A100-evaluation/TDC-LAYERS-ORACLE/template_benchmark_cudnn.template:396). */
#define TDC_W_KCRS 0
#define TDC_W_CRSK 1

/* Epilogue flags for tdc_conv2d_f32. */
#define TDC_EPI_NONE 0
#define TDC_EPI_RELU 1

/*
 * Tiling parameters.  th, tw, tc keep the meaning of the reference generators' TH, TW,
 * TC macros (template_benchmark_cudnn.template:14-16; gen_from_occupancy.py:113-139):
 * output rows per thread, output columns per thread, input channels staged per chunk.
 * The reference fixes "one output channel per thread, all N channels per block"; on
 * B200 those two become parameters (tn, nog), and a CTA may own several images of a
 * small feature map (imgs), split the staged channels over ks thread slices, and split
 * the channel chunks over the kc CTAs of a thread-block cluster; partial sums are reduced
 * in (distributed) shared memory in a fixed order (no atomics).
 * A field left 0 is chosen by tdc_select_tile.
 */
typedef struct tdc_tile {
    int th;   /* output rows per thread                (1 or 2)                    */
    int tw;   /* output columns per thread             (4, 7 or 8)                 */
    int tc;   /* input channels per staged chunk       (multiple of ks)            */
    int tn;   /* output channels per thread            (4 or 8)                    */
    int nog;  /* output-channel groups per CTA         (CTA covers tn*nog channels)*/
    int gy;   /* thread rows per CTA per image         (CTA covers gy*th rows)     */
    int gx;   /* thread columns per CTA per image      (CTA covers gx*tw columns)  */
    int imgs; /* images per CTA (>1 only if gy,gx cover the whole output map)      */
    int ks;   /* channel slices per CTA (in-CTA split of the reduction)            */
    int kc;   /* CTAs per thread-block cluster that share one output tile, each    *
               * walking a range of channel chunks; summed over distributed shared  *
               * memory in rank order (1..8; 1 = no cluster)                        */
} tdc_tile;

/* What the selector needs to know about a device; fill with tdc_query_device or by
 * hand (the analytical model of TDC-LAYERS-MODELING/model.py:264-265 takes the same
 * kind of constants: num_sm, num_threads). */
typedef struct tdc_devinfo {
    int sm_count;        /* 148 on B200                                  */
    int smem_per_cta;    /* opt-in dynamic shared memory per CTA, bytes  */
    int regs_per_sm;     /* 65536                                        */
    int threads_per_sm;  /* 2048                                         */
} tdc_devinfo;

/* Launch facts of one (shape, tile) pair, for table builders and tests. */
typedef struct tdc_launch_info {
    int    grid_x, grid_y;   /* CTAs                                     */
    int    threads;          /* threads per CTA                          */
    size_t smem_bytes;       /* dynamic shared memory per CTA            */
    int    regs_per_thread;  /* of the kernel variant, from the runtime  */
    int    ctas_per_sm;      /* occupancy API result                     */
} tdc_launch_info;

TDC_API const char* tdc_last_error_string(void);
TDC_API int         tdc_version(void);

/* Device facts. No counterpart in the reference (constants are hard-coded at
 * A100-evaluation/TDC-LAYERS-MODELING/model.py:264-265). device < 0 = current. */
TDC_API int tdc_query_device(int device, tdc_devinfo* out);

/*
 * The hot path: y = cross-correlation(x, w), zero padding, no bias.
 * Stands in for (1) the core step of TKConv2dC.forward, F.conv2d(out, core_kernel,
 * None, stride, padding) at inference/TKConv.py:92-93, and (2) the reference kernel
 * conv2d(float* input, const float* kernel, float* outputs) with its launch
 * <<<TCS*THS, N*TWS, smem>>> at template_benchmark_cudnn.template:365-402,490-492.
 * Differences a caller can rely on: any batch, stride 1 or 2, R=S in {1,3} on the fast
 * path and any R,S <= 7 on the generic path, y need NOT be zeroed first (the reference
 * kernel accumulates with atomicAdd into a zeroed buffer), results are run-to-run
 * bit-identical for a given tile.
 *   x [B][C][H][W], w per w_layout, y [B][K][Ho][Wo]; tile may be NULL (auto).
 */
TDC_API int tdc_core_conv2d_f32(const float* x, const float* w, float* y,
                        int B, int C, int H, int W, int K, int R, int S,
                        int pad, int stride, int w_layout,
                        const tdc_tile* tile, void* stream);

/* Same conv with the epilogue of the last 1x1 step of TKConv2dC.forward,
 * F.conv2d(out, last_kernel, bias) at inference/TKConv.py:94 (bias may be NULL), and
 * an optional ReLU (the Activation that follows a block's BatchNorm,
 * A100-evaluation/EndToEnd/resnet18-tk/src/BasicBlock.cu:44-51). */
TDC_API int tdc_conv2d_f32(const float* x, const float* w, const float* bias, float* y,
                   int B, int C, int H, int W, int K, int R, int S,
                   int pad, int stride, int w_layout, int epilogue,
                   const tdc_tile* tile, void* stream);

/* Epilogue of the *_epi entry points:  y = relu?( conv * scale[k] + bias[k] + residual ).
 * It is what follows a Tucker conv in the reference's blocks, folded into the last launch:
 * the bias of TKConv.py:94, an inference-mode BatchNorm as a per-channel scale and shift
 * (BatchNorm.cu:54-71 of the end-to-end skeleton; bn1/bn2 at inference/resnet_inet_tt.py:105-110),
 * the residual add and the ReLU (resnet_inet_tt.py:112-115).  Any pointer may be NULL. */
typedef struct tdc_epilogue {
    const float* scale;     /* [K]                                         */
    const float* bias;      /* [K]                                         */
    const float* residual;  /* [B][K][Ho][Wo], same layout as y            */
    int          relu;      /* != 0: max(.,0) last                         */
} tdc_epilogue;

TDC_API int tdc_conv2d_epi_f32(const float* x, const float* w, float* y,
                   int B, int C, int H, int W, int K, int R, int S,
                   int pad, int stride, int w_layout, const tdc_epilogue* epi,
                   const tdc_tile* tile, void* stream);

/* KCRS -> CRSK, once per weight load.  Replaces nothing in the reference (its drivers
 * fill k[c][r][s][n] with ones directly, template_benchmark_cudnn.template:425-428);
 * needed because TKConv.py stores core_kernel as [R2][R1][kh][kw]. */
TDC_API int tdc_permute_weights(const float* w_kcrs, float* w_crsk,
                        int K, int C, int R, int S, void* stream);

/*
 * Tile selection.  Stands in for the analytical selector modeling()/build_table() of
 * A100-evaluation/TDC-LAYERS-MODELING/model.py:135-234 (same cost terms: filter, input
 * and output volumes and a flops*waves latency term), re-derived for B200's SM count,
 * shared memory and register file.  dev may be NULL (current device is queried).
 */
TDC_API int tdc_select_tile(int B, int C, int H, int W, int K, int R, int S,
                    int pad, int stride, const tdc_devinfo* dev, tdc_tile* out);

/* Completes the zero fields of *tile for the shape, checks it against the device and
 * reports the launch it would produce (no launch happens).  The reference computes the
 * same facts in its occupancy probe, A100-evaluation/Gen-occupancy/template.cu:278-285. */
TDC_API int tdc_tile_info(int B, int C, int H, int W, int K, int R, int S, int pad, int stride,
                  tdc_tile* tile, tdc_launch_info* info);

/* Modelled cost (arbitrary units, lower is better) of a completed tile: the quantity
 * tdc_select_tile minimises.  Mirrors build_table's (K, I, O, flops*waves) tuple,
 * model.py:157-184; vols[0..3] receive those four terms when vols != NULL. */
TDC_API int tdc_tile_cost(int B, int C, int H, int W, int K, int R, int S, int pad, int stride,
                  const tdc_tile* tile, const tdc_devinfo* dev, double* cost, double* vols);

/*
 * The Tucker block of TKConv2dC.forward, inference/TKConv.py:90-95:
 *   z1 = conv1x1(x, w1[R1][C]);  z2 = conv(z1, wcore, stride, pad);
 *   y  = conv1x1(z2, w3[K][R2]) + bias.
 * Also the TkConv::forward chain conv1->conv2->conv3 of
 * A100-evaluation/EndToEnd/resnet18-tk/src/BasicBlock.cu:27-32.
 * The two intermediates live in `workspace` (tdc_tk_block_workspace_bytes), which is
 * sized to stay resident in B200's L2 for the benchmark shapes; the three steps run
 * back to back on `stream`.  w1 is [R1][C], w3 is [K][R2] (torch 1x1 layouts), wcore per
 * w_layout.  bias may be NULL.  epilogue as in tdc_conv2d_f32.
 */
TDC_API size_t tdc_tk_block_workspace_bytes(int B, int C, int H, int W, int R1, int R2, int K,
                                    int R, int S, int pad, int stride);
TDC_API int tdc_tk_block_f32(const float* x, const float* w1, const float* wcore, const float* w3,
                     const float* bias, float* y,
                     int B, int C, int H, int W, int R1, int R2, int K, int R, int S,
                     int pad, int stride, int w_layout, int epilogue,
                     const tdc_tile* core_tile /* NULL = auto */,
                     void* workspace, size_t workspace_bytes, void* stream);

/* tdc_tk_block_f32 with the full epilogue on its last step (epi may be NULL). */
TDC_API int tdc_tk_block_epi_f32(const float* x, const float* w1, const float* wcore, const float* w3, float* y,
                     int B, int C, int H, int W, int R1, int R2, int K, int R, int S,
                     int pad, int stride, int w_layout, const tdc_epilogue* epi,
                     const tdc_tile* core_tile /* NULL = auto */,
                     void* workspace, size_t workspace_bytes, void* stream);

/*
 * The Tucker block for callers that must not allocate device memory.  No counterpart in the
 * reference (its layers cudaMalloc whatever they need when they are initialised).
 *
 * Who needs it: code that runs where cudaMalloc is off the table — a serving loop whose
 * whole memory budget was handed to one arena at start-up, a plug-in living inside a host
 * framework that owns the allocator and forbids side allocations, a step that may only
 * enqueue work on a stream.  tdc_tk_block_f32 asks such a caller for a workspace it has no
 * way to produce.  This variant keeps the two intermediates (z1, z2) in a fixed array that
 * is part of the library image instead: TDC_STATIC_WORKSPACE_BYTES of device memory that a
 * GPU holds from the moment the library's code is loaded onto it until the process exits.
 * With CUDA's lazy module loading (the default) that moment is the first call of this
 * library on the device; with CUDA_MODULE_LOADING=EAGER it is context creation.  Either
 * way the memory is claimed by the driver when it loads the module, not by this function.
 *
 * Same arguments, results and status codes as tdc_tk_block_f32 minus the workspace pair; the
 * caller still passes x, the factors and y.  It returns TDC_ERR_WORKSPACE, with the needed and
 * the available byte counts in the message, when tdc_tk_block_workspace_bytes(...) for the shape
 * exceeds TDC_STATIC_WORKSPACE_BYTES.  It performs no cudaMalloc/cudaFree and calls nothing that
 * does.
 *
 * Set-up: the first call on each device looks up the array's device address (once, with that
 * device current), which is also when a lazily loaded module lands on the device.  Make that
 * first call during start-up — before any stream capture begins and before the host
 * application's arena takes the rest of the device memory, or the module load itself can
 * fail for lack of memory (reported as TDC_ERR_CUDA).
 *
 * Sharing: all calls on a device use the same array and it keeps whatever the previous call
 * left there; both intermediates are fully overwritten before they are read, so nothing needs
 * clearing.  Two calls that overlap on the GPU (different streams, or different host threads
 * without ordering between their streams) race on it — serialise them.
 */
#define TDC_STATIC_WORKSPACE_BYTES (32u << 20)   /* 32 MiB: every benchmark Tucker block up to batch 32 */
TDC_API int tdc_tk_block_f32_static(const float* x, const float* w1, const float* wcore, const float* w3,
                     const float* bias, float* y,
                     int B, int C, int H, int W, int R1, int R2, int K, int R, int S,
                     int pad, int stride, int w_layout, int epilogue,
                     const tdc_tile* core_tile /* NULL = auto */, void* stream);

/*
 * Tensor-core variant (tcgen05, TF32 operands, fp32 accumulation in tensor memory).  No
 * counterpart in the reference, whose kernel and whose cuDNN calls are fp32 FMA code
 * (template_benchmark_cudnn.template:365-402; inference/TKConv.py:92-93).  Same result
 * definition as tdc_conv2d_epi_f32 for "same" convolutions: R = S in {1, 3}, stride 1,
 * pad = (R-1)/2; a 1x1 filter may also be strided (the down-sampling shortcut of a residual
 * stage, inference/resnet_inet_tt.py:27-29,363-366): `flags` carries stride - 1 in its low four bits,
 * H and W are the input image, y is [B][K][(H-1)/stride+1][(W-1)/stride+1].
 *   mode 3  "3xTF32": operands split into hi + lo TF32 parts, three MMAs per product;
 *           fp32-level accuracy (held to the same 1e-5 bar as the fp32 kernels)
 *   mode 4  "3xFP16": the same split with fp16 parts (the lo part scaled by 2^11 to stay clear of fp16's
 *           subnormals): the same 22 significant bits per operand at twice the MMA rate and half the
 *           accumulations per output, so both faster and closer to fp64 than mode 3; the input and the filter
 *           are scaled by powers of two into fp16's range (see tdc_conv2d_tc_ranged); with TDC_TC_EXACT_RANGE the
 *           prepared filter's scratch tail is used by the call in flight, so such calls sharing one prepared
 *           filter must not overlap on the GPU
 *   mode 1  plain TF32: one MMA per product; 5e-3 bar; reported separately
 * Use: tdc_tc_plan_make once per layer shape, tdc_tc_prepare_weights once per weight load
 * into a caller-owned buffer of plan.weights_bytes, then tdc_conv2d_tc per call.  Every
 * device-side wait is bounded; tdc_tc_status reads (and synchronises for) the device status
 * word: 0 = no wait ever ran out and no mode-4 output was non-finite, 1 = a wait ran out, 2 = a
 * mode-4 launch produced a value that is not finite (input beyond the scaled fp16 range).
 */
typedef struct tdc_tc_plan {
    int    C, K, R, S, mode;
    int    nt;            /* output channels per CTA (MMA N)              */
    int    cb;            /* channels per K step: 8 (TF32), 16 (fp16)     */
    int    nkb, n_ocb;    /* channel blocks, output-channel blocks        */
    int    hl;            /* 2 when operands are split (modes 3, 4), else 1 */
    int    general;       /* 1: made by tdc_tc_plan_make_general, 2: by tdc_tc_plan_make_strided */
    int    stride;        /* strided-row plans: the stride they were made for, else 0 */
    int    phase;         /* strided-row plans: 1 when the column phases count from an even input column (odd padding at stride 2) */
    size_t weights_bytes; /* size of the pre-arranged filter              */
} tdc_tc_plan;

TDC_API const char* tdc_tc_last_error_string(void);
TDC_API int tdc_tc_plan_make(int C, int K, int R, int S, int mode, tdc_tc_plan* out);
/* A plan for ANY filter size, stride and padding (the 7x7 stride-2 stem, the 3x3 stride-2 cores of the
 * down-sampling blocks: inference/resnet_inet_tt.py:319-320,32-38): the contraction runs over
 * (channel, filter row, filter column) triples gathered by the loaders, i.e. a classic implicit GEMM
 * that re-reads the input R*S/stride^2 times from cache.  Stride and padding come with the call. */
TDC_API int tdc_tc_plan_make_general(int C, int K, int R, int S, int mode, tdc_tc_plan* out);
/* The gathering plan for STRIDED convolutions whose filter is 2 or 4 strides wide (3x3 stride 2: the down-sampling cores;
 * 7x7 stride 2: the stem, inference/resnet_inet_tt.py:319-320), mode 4.  Input column ox*stride - pad + dx is written
 * as dx = j*stride + p: the phase p joins (channel, filter row) in the contraction, and the step j becomes a TAP — a
 * shift by j output positions, which costs no copy at all.  The loaders then gather C*R*stride values per position
 * instead of C*R*S (42 instead of 147 for the stem).  At stride 2 the two phases of a (channel, filter row) are
 * neighbours in memory; the plan counts them from an even input column (with an odd padding the filter's first column
 * becomes a tap one position to the left), so that one 8-byte copy fetches both when the image is an even number of
 * pixels wide and x is 16-byte aligned (4-byte copies otherwise).  nt = 0: the default block size.  Stride and the
 * parity of the padding are part of the plan; the call repeats stride and padding in `flags`. */
TDC_API int tdc_tc_plan_make_strided(int C, int K, int R, int S, int stride, int pad, int mode, int nt, tdc_tc_plan* out);
/* Output channels per block are 128 / 64 / 32 by K in the plans above, which suits layers with many output positions.
 * tdc_tc_pick_nt gives the block size for a layer with `positions` output positions (B x padded image; smaller blocks
 * mean more CTAs when the positions alone do not fill `sm_count` SMs), tdc_tc_plan_make_nt makes a plan (general or
 * not) with that block size; its prepared filter differs, so a caller keeps one per block size it uses. */
TDC_API int tdc_tc_pick_nt(int K, int mode, long long positions, int sm_count);
TDC_API int tdc_tc_plan_make_nt(int C, int K, int R, int S, int mode, int general, int nt, tdc_tc_plan* out);
TDC_API int tdc_tc_prepare_weights(const tdc_tc_plan* plan, const float* w, int w_layout, void* wt, void* stream);
#define TDC_TC_STRIDE_MASK 0x0F  /* flags & mask = stride - 1 (1x1 filters and general plans)         */
#define TDC_TC_PAD_MASK    0xF0  /* (flags & mask) >> 4 = padding (general plans); other bits must be 0 */
#define TDC_TC_PAD_SHIFT   4
#define TDC_TC_EXACT_RANGE 0x100 /* mode 4: find max|x| with a pass over x instead of sampling it (see tdc_conv2d_tc_ranged) */
/* Modes 3 and 4: the tensor core truncates its fp32 running sum toward zero at every accumulation, so a sum of n
 * accumulations comes out n * 2^-26 too small on average.  With this flag the epilogue puts that expected loss back
 * (one factor 1 + n * 2^-26 on the main accumulator): the error left has no sign and no longer adds up through the
 * layers of a network (the assemblies and the Tucker module set it).  Without it the sums are stored as the tensor
 * core returns them: sums of small integers, where nothing is truncated, are exact, which is what the reference
 * drivers check (template_benchmark_cudnn.template:404-411,489-498). */
#define TDC_TC_UNBIASED    0x200
/* Stream order is kept as with any launch.  (The persistent kernel is launched with programmatic stream serialization:
 * its CTAs may be scheduled while the kernel before it in the stream still runs, and wait inside, before they touch any
 * global memory but the filter plan's constants, until that kernel has completed and its writes are visible.  A caller
 * sees nothing of it but shorter gaps between launches; it also holds under stream capture into a CUDA graph.) */
TDC_API int tdc_conv2d_tc(const tdc_tc_plan* plan, const float* x, const void* wt, float* y,
                          int B, int H, int W, const tdc_epilogue* epi, int flags, void* stream);
/* Mode 4 scales the input by a power of two into fp16's range (which ends at 65504) and undoes the scaling in the
 * epilogue.  fp16 keeps its 11 significant bits over 30 binades, so the scale need only be roughly right:
 *   - by default every CTA of the kernel samples 1500 - 2000 elements spread over x and puts the largest at 2^8, which
 *     leaves a factor of 256 for values the sample missed (no extra launch; the loads run under the CTA's start-up);
 *   - with TDC_TC_EXACT_RANGE in `flags` a pass over all of x finds the true maximum first (one more launch);
 *   - a caller that chains layers (the three steps of TKConv2dC.forward, inference/TKConv.py:90-95) has the bound
 *     for free: y_absmax, when given, receives the partial maxima of |y| (TDC_TC_ABSMAX_FLOATS floats, every entry
 *     written), and the next call takes the same buffer as x_absmax (it must bound the x of THAT call; a bound over
 *     more data only costs precision).
 * An input that leaves fp16's range all the same (more than 256 times the sampled maximum, or not finite) makes
 * outputs that are not finite; the kernel sees them and sets the status word that tdc_tc_status reads to 2.
 * Other modes ignore x_absmax and refuse y_absmax. */
#define TDC_TC_ABSMAX_FLOATS 1024
TDC_API int tdc_conv2d_tc_ranged(const tdc_tc_plan* plan, const float* x, const void* wt, float* y,
                          int B, int H, int W, const tdc_epilogue* epi, int flags,
                          const float* x_absmax, float* y_absmax, void* stream);
/* Whether tdc_conv2d_tc can launch this plan on images of H x W (TDC_OK), without launching: wide images with many
 * output channels per block may not leave room for two stages in shared memory (TDC_ERR_SMEM); a plan with a smaller
 * block (tdc_tc_plan_make_nt) then fits.  The prepared filter depends on the block size, so ask before preparing. */
TDC_API int tdc_tc_check_launch(const tdc_tc_plan* plan, int B, int H, int W, int flags);
TDC_API int tdc_tc_status(int* out);

/*
 * Pooling layer of the end-to-end skeleton: Pool::initialize(b,c,h,w,pad,windowH,windowW,mode,stride) /
 * Pool::forward (A100-evaluation/EndToEnd/resnet18-tk/src/Pool.cu:8-48, a cudnnPoolingForward call; the
 * nn.MaxPool2d(3,2,1) of inference/resnet_inet_tt.py:323).  x [B][C][H][W] -> y [B][C][Ho][Wo] with
 * Ho = (H - window_h + 2*pad)/stride + 1; padding never wins a maximum; NaNs are not propagated
 * (CUDNN_NOT_PROPAGATE_NAN there).  Needs 2*pad <= window so that no window is all padding.
 */
#define TDC_POOL_MAX              0
#define TDC_POOL_AVG_INCLUDE_PAD  1
#define TDC_POOL_AVG_EXCLUDE_PAD  2
TDC_API int tdc_pool2d_f32(const float* x, float* y, int B, int C, int H, int W, int window_h, int window_w,
                           int pad, int stride, int mode, void* stream);

/*
 * Per-channel scale, shift and ReLU with image strides: y[b][c][i] = relu?(x[b][c][i]*scale[c] + shift[c]) for
 * i < HW, image b of x at x + b*x_image_stride and of y at y + b*y_image_stride (strides in elements,
 * >= C*HW).  One call stands for the reference's BatchNorm::forward in its inference form followed by
 * Activation::forward (A100-evaluation/EndToEnd/densenet121-tk/src/BatchNorm.cu:58-80, src/Activation.cu:38-41)
 * ahead of each conv of a dense layer (src/TenDense.cu:44-53; norm1 / norm2 of
 * inference/densenet_inet_tt.py:36-60), reading the first C channels of the block's feature buffer in place;
 * with scale = shift = NULL and relu = 0 it is the strided copy that appends a layer's new features to that
 * buffer (Concate::forward, inc/common.h:165-177).  scale / shift NULL = 1 / 0.
 */
TDC_API int tdc_affine_relu_f32(const float* x, float* y, const float* scale, const float* shift, int B, int C, int HW,
                                long long x_image_stride, long long y_image_stride, int relu, void* stream);

/*
 * Layer objects with the surface of the reference's end-to-end classes:
 * Conv::initialize(b,c,h,w,n,pad,r,s,stride,weightFile,use_bias) / float* Conv::forward(float*)
 * (A100-evaluation/EndToEnd/resnet18-tk/inc/common.h:38-69, src/Conv.cu:2-125) and
 * TkConv::initialize(C,N1,N2,N3,h,w,...,down_sample) / forward (common.h:158-166,
 * src/BasicBlock.cu:15-32).  As there, a layer owns its weights and its output buffer
 * and forward() returns that buffer; unlike there, weights are supplied by the caller
 * (HOST pointers, KCRS; NULL = all ones as the reference fills them), errors come back
 * as status codes, and destroy() frees what create() allocated.
 * The *_host variants take HOST input/output: copy in, run, copy out, synchronise — the
 * shape of the per-shape drivers' main() (template_benchmark_cudnn.template:412-498).
 */
typedef struct tdc_conv   tdc_conv;
typedef struct tdc_tkconv tdc_tkconv;

TDC_API int  tdc_conv_create(tdc_conv** out, int b, int c, int h, int w, int n, int pad,
                     int r, int s, int stride, const float* host_w_kcrs,
                     const float* host_bias /* NULL = no bias */);
TDC_API int  tdc_conv_set_tile(tdc_conv* l, const tdc_tile* tile);
/* 0: fp32 FMA kernels (default); 3 / 1: tensor cores, 3xTF32 / TF32 (stride-1 1x1 and 3x3 "same" layers). */
TDC_API int  tdc_conv_set_precision(tdc_conv* l, int mode);
TDC_API int  tdc_conv_forward(tdc_conv* l, const float* dev_in, float** dev_out, void* stream);
TDC_API int  tdc_conv_forward_host(tdc_conv* l, const float* host_in, float* host_out);
/* The same without the final synchronise, on `stream`: independent layers (the per-shape drivers of a sweep) run
 * on streams of their own, so the copy in of one overlaps the copy out of another.  Host buffers must be pinned
 * for the copies to be asynchronous; the caller synchronises the stream before reading host_out. */
TDC_API int  tdc_conv_forward_host_async(tdc_conv* l, const float* host_in, float* host_out, void* stream);
TDC_API void tdc_conv_destroy(tdc_conv* l);

TDC_API int  tdc_tkconv_create(tdc_tkconv** out, int b, int C, int N1, int N2, int N3, int h, int w,
                       int r, int s, int pad, int stride,
                       const float* host_w1, const float* host_wcore_kcrs,
                       const float* host_w3, const float* host_bias);
/* 0: the three fp32 launches of tdc_tk_block_f32 (default).  1 / 3 / 4: ONE tensor-core launch (tdc_conv2d_tc in that
 * mode) on the filter w[k][c][i][j] = sum w3[k][r2] * core[r2][r1][i][j] * w1[r1][c], merged on the host in double and
 * rounded once — the weight TKConv2dR recovers before its single conv (inference/TKConv.py:310-322).  The same linear
 * map as conv1 -> conv2 -> conv3 of TkConv::forward (src/BasicBlock.cu:27-32) with neither intermediate ever formed;
 * more multiply-adds, yet faster on this GPU while the three steps are bound by launches and memory passes. */
TDC_API int  tdc_tkconv_set_precision(tdc_tkconv* l, int mode);
TDC_API int  tdc_tkconv_forward(tdc_tkconv* l, const float* dev_in, float** dev_out, void* stream);
TDC_API int  tdc_tkconv_forward_host(tdc_tkconv* l, const float* host_in, float* host_out);
TDC_API void tdc_tkconv_destroy(tdc_tkconv* l);

#ifdef __cplusplus
}
#endif
#endif /* TDC_B200_H */
