// Persistent form of the tensor-core convolution kernel (included by conv_tc.cu, which holds
// the description of the algorithm, the operand layouts and the helpers used here).
//
// One CTA per SM walks a list of tiles (tile = MT x 128 positions x NT output channels).
// What a one-tile-per-CTA launch pays per tile — tensor-memory allocation, barrier set-up, a
// cold first load, and an epilogue during which the tensor core idles — is paid once or hidden:
//   * loaders (warps 0-7) never stop: the shared-memory stages and the raw-input ring behind them
//     run across tile boundaries, so the first channel blocks of the next tile are staged while
//     the MMAs of this one finish;
//   * the accumulators of a CTA tile are handed over one 128-position tile at a time: warp 8+mt
//     issues the MMAs of position tile mt and may start the next CTA tile as soon as ITS
//     accumulators have been read, while the other issuers still work on this one (and tensor
//     memory holds two CTA tiles outright when 2 x MT x columns-per-tile fits in 512 columns);
//   * four groups of four epilogue warps (12-27) take the (position tile, 16-channel chunk)
//     items of a CTA tile in turn; an accumulator is handed back as soon as all its chunks are in
//     registers, before the stores.
//
// Runs.  The tensor core rounds its running sum at every accumulation, so the error of a tile grows with
// the number of MMAs that feed one accumulator.  The host may therefore cut the channel blocks of a tile
// into `nseg` runs: every run starts fresh accumulators, and the epilogue adds the runs to y in fp32 (the
// thread that stored a partial sum is the one that reads it back).  Long contractions land on small
// feature maps, where the extra pass over y is cheap.
//
// Input loaders (template parameter LD):
//   0  ring:  global -> 4-byte cp.async -> raw fp32 slots -> registers -> split -> operand layout; a thread
//             converts the rows it copied, so cp.async.wait_group is all the synchronisation the ring needs;
//   1  vec:   1x1 filters, 16-byte global loads into registers (TF32 operands only);
//   2  bulk:  a producer thread (warp 11) issues cp.async.bulk.tensor boxes of 32 pixels x 16 channels of
//             this GPU's own input into raw slots, completion on an mbarrier per slot; warps 0-7 only convert.
//             No load instruction is issued per element, which is what bounds loader 0 (fp16 operands,
//             images of a multiple of 4 pixels, 16-byte aligned input).
// Every mbarrier wait is bounded; a wait that runs out raises the CTA's abort flag, every
// role leaves its loop at the next check, the status word is set and tensor memory is freed.
#pragma once

namespace tdc_tc {

// A CTA is 28 warps: LW loader warps (8 or 12, a template parameter), 4 issuer warps (one lane each), and what is left
// as groups of four epilogue warps (4 or 3 groups).  LW is a multiple of 4, so the epilogue warps that follow the
// issuers read the lane quarter warp % 4 of tensor memory.  Which split a call takes follows from its epilogue, a
// latency chain per work item (tensor memory -> registers -> scale, shift, residual, ReLU -> stores): a launch that
// carries those options wants the four groups, a launch that only stores (the first two steps of a Tucker chain, a
// bare layer) is paced by its loaders and takes the twelve loader warps.  Measured on one GPU in one run, batch 256 /
// 64 / 128: TK-ResNet-18 4.10 ms, TK-ResNet-50 5.17 ms, a TK-VGG-16 chunk 10.4 ms with the split chosen per call;
// 4.11 / 5.13 / 10.9 with 8 loader warps for every launch; 4.18 / 5.45 / 11.0 with 12 for every launch; 4.35 / 5.57 /
// 10.7 with the earlier two groups of 32-channel items (640 threads at 96 registers).  The bare sweep layers are level
// in all of these (365 .. 368 us over the eight); the gathering plans gain a tenth from the twelve (stem 484 -> 436 us).
// The loader count is a compile-time constant because it sizes the per-thread row arrays (one or two rows with 384
// loaders where 256 need two to four); as a launch parameter of one kernel the twelve gained nothing.
// Work items are 16 channels wide so that 72 registers per thread hold them without spills.
constexpr int P_WARPS   = 28;
constexpr int P_THREADS = 32 * P_WARPS;
constexpr int P_EPI_W   = 16;           // channels an epilogue thread holds at a time
// patch rows a CTA may stage (3x3 filters: MT x 128 positions plus two image rows of halo, images up to 256 wide)
__host__ __device__ constexpr int p_rows_cap(int mt) { return mt == 1 ? 768 : 1024; }
constexpr int P_HEADER  = 1024;  // bytes of barriers, flags and the producer's box table in front of the stages
constexpr int P_MAXBOX  = 64;    // boxes one raw slot may hold (entries of the box table)
constexpr int LD_RING = 0, LD_VEC = 1, LD_BULK = 2;

// Tile t of the list -> first output position, position tiles it holds (`cnt` <= MT), output-channel block.
// Tiles of the complete rounds hold MT position tiles; what is left for the last, partial round is spread over
// all CTAs as smaller tiles (with one output-channel block; a.full_groups covers every tile otherwise), so the
// launch ends after a part of a round instead of a whole one.
template <int MT>
__device__ __forceinline__ void tile_of(const Args& a, long long t, long long& g0, int& cnt, int& ocb) {
    long long tg = t;
    ocb = 0;
    if (a.n_ocb > 1) { tg = a.small ? (long long)fastdiv((uint32_t)t, a.fd_nocb) : t / a.n_ocb; ocb = (int)(t - tg * a.n_ocb); }
    if (tg < a.full_groups) { g0 = tg * (MT * M_TILE); cnt = MT; return; }
    const long long first = a.tail_first_pt + (tg - a.full_groups) * a.tail_cnt, left = a.pt_total - first;
    g0 = first * M_TILE;
    cnt = left < a.tail_cnt ? (int)left : a.tail_cnt;
}

// Image of padded position g (0 <= g < total_pos + Lp), and row of position `rem` within a padded image.  Position counts
// fit 31 bits for every layer of practical size (`small`), and then a division is a multiply and a shift (FastDiv): the
// per-tile index arithmetic of the loaders and the producer and the per-item arithmetic of the epilogue are made of these.
__device__ __forceinline__ long long image_of(const Args& a, long long g) {
    return a.small ? (long long)fastdiv((uint32_t)g, a.fd_Lp) : g / a.Lp;
}
__device__ __forceinline__ int row_of(const Args& a, int rem) {
    return a.small ? (int)fastdiv((uint32_t)rem, a.fd_Wp) : rem / a.Wp;
}

// The pixels of image b that the patch [gp0, gp0 + rows) of padded positions needs: the run starts at pixel
// `pix4` (rounded down to a 16-byte boundary, which a bulk-tensor copy must start on) and takes `nbox` boxes
// of BOXW pixels; nbox = 0 when the patch meets only padding of that image.  Producer and converters call
// this with the same arguments, so they agree on where every pixel lands in a raw slot.
__host__ __device__ __forceinline__ void image_run(int H, int W, int Wp, int Lp, long long gp0, int rows, long long b, int& pix4, int& nbox) {
    const long long img0 = b * Lp;
    const int ls = gp0 > img0 ? (int)(gp0 - img0) : 0;
    const int le = gp0 + rows < img0 + Lp ? (int)(gp0 + rows - img0) : Lp;     // local padded positions [ls, le)
    nbox = 0; pix4 = 0;
    if (le <= ls) return;
    int y0 = ls / Wp, x0 = ls - y0 * Wp;
    if (x0 >= W) { ++y0; x0 = 0; }                                             // starts on the zero column
    int y1 = (le - 1) / Wp, x1 = (le - 1) - y1 * Wp;
    if (y1 >= H) { y1 = H - 1; x1 = W - 1; } else if (x1 >= W) x1 = W - 1;      // ends on the zero row / column
    if (y0 >= H) return;
    const int ps = y0 * W + x0, pe = y1 * W + x1 + 1;
    if (pe <= ps) return;
    pix4 = ps & ~3;
    nbox = (pe - pix4 + BOXW - 1) / BOXW;
}

// The same on the device, dividing by multiplication.
__device__ __forceinline__ void image_run(const Args& a, long long gp0, int rows, long long b, int& pix4, int& nbox) {
    const int H = a.H, W = a.W, Wp = a.Wp, Lp = a.Lp;
    const long long img0 = b * Lp;
    const int ls = gp0 > img0 ? (int)(gp0 - img0) : 0;
    const int le = gp0 + rows < img0 + Lp ? (int)(gp0 + rows - img0) : Lp;
    nbox = 0; pix4 = 0;
    if (le <= ls) return;
    int y0 = row_of(a, ls), x0 = ls - y0 * Wp;
    if (x0 >= W) { ++y0; x0 = 0; }
    int y1 = row_of(a, le - 1), x1 = (le - 1) - y1 * Wp;
    if (y1 >= H) { y1 = H - 1; x1 = W - 1; } else if (x1 >= W) x1 = W - 1;
    if (y0 >= H) return;
    const int ps = y0 * W + x0, pe = y1 * W + x1 + 1;
    if (pe <= ps) return;
    pix4 = ps & ~3;
    nbox = (pe - pix4 + BOXW - 1) / BOXW;
}

__device__ __forceinline__ void bulk_tensor_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}

// Measurement builds (not compiled otherwise); tdc_tc_profile_read hands g_tc_prof to the host.
//   -DTDC_TC_PROFILE=1  phases of a CTA and the issuers' waits only, which leaves the kernel's timing as it is: per CTA
//                       that has a tile, the clocks from its start to the end of the set-up [16], to its first full stage
//                       [17], to the end of its first issuer [18] and to its last barrier [19], and the CTAs counted [20];
//                       within the start-up: to the producer's first copy issued [21] (bulk loader), to the end of the
//                       loaders' first index work [22] and to their first raw block landed [23];
//                       per stage use of an issuer the clocks spent issuing it [10] and the uses counted [11];
//   -DTDC_TC_PROFILE=2  also every role's waits and spans [0, 12) and role totals [12, 16): the clock reads in the
//                       loaders' loops slow the kernel by a third or more, so only the shares within a role mean something.
#ifdef TDC_TC_PROFILE
__device__ unsigned long long g_tc_prof[24];
#define TDC_PROF_LIGHT(kind) ((kind) == 3 || (kind) == 4)            /* the issuers' two waits */
#define TDC_PROF_DECL long long prof_t[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0}; const long long prof_start = clock64(); bool prof_first = true
#define TDC_PROF_WAIT(kind, call) ([&]() { if (TDC_TC_PROFILE < 2 && !TDC_PROF_LIGHT(kind)) return (bool)(call); \
                                           const long long t0_ = clock64(); const bool ok_ = (call); prof_t[kind] += clock64() - t0_; return ok_; }())
#define TDC_PROF_SPAN_BEGIN const long long span0_ = TDC_TC_PROFILE < 2 ? 0 : clock64()
#define TDC_PROF_SPAN_END(kind) do { if (TDC_TC_PROFILE >= 2) prof_t[kind] += clock64() - span0_; } while (0)
#define TDC_PROF_FLUSH(role) do { if (lane == 0 && (TDC_TC_PROFILE >= 2 || (role) == 2)) { \
                                  for (int k_ = 0; k_ < 12; ++k_) if (prof_t[k_]) atomicAdd(&g_tc_prof[k_], (unsigned long long)prof_t[k_]); \
                                  atomicAdd(&g_tc_prof[12 + (role)], (unsigned long long)(clock64() - prof_start)); } } while (0)
#define TDC_PROF_ISSUE_BEGIN const long long issue0_ = clock64()
#define TDC_PROF_ISSUE_END do { prof_t[10] += clock64() - issue0_; prof_t[11] += 1; } while (0)
/* a phase mark by one thread of a CTA that has a tile (`once`: only the first time this thread comes by) */
#define TDC_PROF_MARK(slot, cond, once) do { if ((cond) && blockIdx.x < ntiles && (!(once) || prof_first)) { if (once) prof_first = false; \
                                             atomicAdd(&g_tc_prof[slot], (unsigned long long)(clock64() - prof_cta0)); } } while (0)
#define TDC_PROF_COUNT(slot, cond) do { if ((cond) && blockIdx.x < ntiles) atomicAdd(&g_tc_prof[slot], 1ull); } while (0)
#define TDC_PROF_CTA_START const long long prof_cta0 = clock64()
#else
#define TDC_PROF_DECL
#define TDC_PROF_WAIT(kind, call) (call)
#define TDC_PROF_SPAN_BEGIN
#define TDC_PROF_SPAN_END(kind)
#define TDC_PROF_FLUSH(role)
#define TDC_PROF_ISSUE_BEGIN
#define TDC_PROF_ISSUE_END
#define TDC_PROF_MARK(slot, cond, once)
#define TDC_PROF_COUNT(slot, cond)
#define TDC_PROF_CTA_START
#endif

template <int NT, int MT, int TAPS, int LD, bool F16, int LW = 8>
__global__ void __launch_bounds__(P_THREADS) conv_tc_persist_kernel(const Args a, const __grid_constant__ CUtensorMap tmap) {
    static_assert(LD != LD_VEC || (TAPS == 1 && !F16), "the 16-byte register loader serves 1x1 filters with TF32 operands");
    static_assert(LD != LD_BULK || (F16 && MT <= 2), "the bulk loader converts to fp16 parts; its producer is issuer warp 3, free when MT <= 2");
    constexpr int CBK = KStep<F16>::CH;                               // channels per block
    // the roles of this instantiation (see the top of the file)
    static_assert(LW == 8 || LW == 12, "8 loader warps and four epilogue groups, or 12 and three");
    constexpr int P_LOADERS = LW * 32, P_IW0 = LW, P_EW0 = LW + 4, P_GROUPS = (P_WARPS - P_EW0) / 4, P_PRODUCER = P_IW0 + 3;
    TDC_PROF_CTA_START;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    uint64_t* full_bar   = reinterpret_cast<uint64_t*>(smem_raw);    // [ns]  patch stored + filter landed
    uint64_t* empty_bar  = full_bar + 4;                              // [ns]  MMAs that read the stage are done
    uint64_t* tfull_bar  = empty_bar + 4;                             // [nbuf*MT] the accumulators of a 128-position tile are complete
    uint64_t* tempty_bar = tfull_bar + 8;                             // [nbuf*MT] the epilogue has read them
    uint64_t* rfull_bar  = tempty_bar + 8;                            // [depth] bulk loader: the boxes of a raw slot have landed
    uint64_t* rempty_bar = rfull_bar + 8;                             // [depth] ... and have been converted
    uint32_t* tmem_slot  = reinterpret_cast<uint32_t*>(rempty_bar + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    unsigned int* max_word = reinterpret_cast<unsigned int*>(tmem_slot + 2);   // block-wide maximum: of |x| (given bounds) at the start, of |y| at the end
    unsigned int* range_word = reinterpret_cast<unsigned int*>(tmem_slot + 3); // largest sampled |x|
    int2*     box_tab    = reinterpret_cast<int2*>(smem_raw + 512);   // producer only: (first pixel, image) of each box
    float*    stage0     = reinterpret_cast<float*>(smem_raw + P_HEADER);

    // patch rows per loader thread: MT x 128 positions, plus two image rows of halo for a 3x3 filter (the host keeps
    // the patch within PPT x 256 rows; images up to 256 wide)
    constexpr int PPT = TAPS == 1 ? (MT * M_TILE + P_LOADERS - 1) / P_LOADERS
                                   : (TAPS == 9 ? (p_rows_cap(MT) + P_LOADERS - 1) / P_LOADERS : (MT * M_TILE + 8 + P_LOADERS - 1) / P_LOADERS);
    // a stage holds a.kps channel blocks (one for 3x3 filters; several for one-tap filters, whose stages would
    // otherwise be all hand-over and no work): [kps input blocks][kps filter blocks]
    const int a_floats = a.hl * CB * a.P, b_floats = a.hl * TAPS * CB * NT, stage_floats = a.kps * (a_floats + b_floats);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int halo_rows = a.halo;                                // patch rows beyond the positions of a tile
    const long long HW = (long long)a.H * a.W;
    const uint32_t b_bytes = (uint32_t)b_floats * 4u;
    const int nbuf = a.nbuf;
    const long long ntiles = a.ntiles;          // position tiles x output-channel blocks
    constexpr int SCALED_THREADS = P_LOADERS + 128 * P_GROUPS;       // the converting and the draining warps
    // the producer's first copy would otherwise wait for the fetch of the tensor map
    if (LD == LD_BULK && tid == P_PRODUCER * 32) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap)) : "memory");

    if (tid == (P_IW0 + 1) * 32) {
        for (int s = 0; s < a.ns; ++s) { mbar_init(&full_bar[s], P_LOADERS / 32 + 1); mbar_init(&empty_bar[s], MT); }   // one arrival per loader warp + the filter's bytes
        for (int b = 0; b < 8; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], 4 * (NT / P_EPI_W)); }   // one per issuer; one per epilogue warp and chunk of channels
        for (int d = 0; d < 8; ++d) { mbar_init(&rfull_bar[d], 1); mbar_init(&rempty_bar[d], P_LOADERS / 32); }    // the producer's arrive + bytes; one per converting warp
        *abort_flag = 0;
        *range_word = 0;
        *max_word = 0;                                   // the largest |y| of this CTA (read after the last barrier)
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == P_IW0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)a.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    // The kernel may have been scheduled before the kernels ahead of it in the stream have finished (programmatic
    // dependent launch): nothing they may have written (x, the bound of |x|, y, the residual) is touched before
    // griddepcontrol.wait, which every thread passes once, here.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");      // the kernel after this one may be scheduled as SMs become free
    TDC_PROF_DECL;
    TDC_PROF_MARK(16, tid == 0, false);
    // fp16 operands: the power of two that brings the input just under 2^15 (2^9 when the range is only sampled), and
    // the factor that undoes it (and the filter's, applied when it was prepared) in the epilogue.  Only the converting
    // and the draining warps need them, and they meet once at named barrier 1: the draining warps at once, the loaders
    // after the index work of their first tile, or after their loop when the CTA has no tile — the producer, the issuers
    // and that index work do not wait for the range.
    float xs = 1.f, inv = 1.f;

    if (warp < P_IW0) {
        // ================= loaders =================
        // no division in these loops: the loaders are bound by instruction latency (two warps per scheduler), so the
        // ring positions are counters that wrap, not quotients of a running index
        int st_idx = 0, st_use = 0, st_k = 0;    // stage being filled, parity of its use count, blocks stored in it
        float* stage_A = nullptr;                // the stage being filled
        // where channel block kb of the current tile goes; its first block of a stage waits for the stage and starts
        // the copy of the stage's filter blocks
        // The filter blocks of the very first stage are asked for before the index work of the first tile (first_filter),
        // so that they land under it; open_stage then skips that copy.
        auto first_filter = [&](const float* wt_tile) {
            if (tid == 0) {
                const uint32_t bytes = (uint32_t)(a.nkb < a.kps ? a.nkb : a.kps) * b_bytes;
                mbar_expect_tx(&full_bar[0], bytes);
                bulk_g2s(stage0 + a.kps * a_floats, wt_tile, bytes, &full_bar[0]);
            }
        };
        // the loaders' side of the meeting at named barrier 1
        auto scale_here = [&]() { if constexpr (F16) xs = range_scale(range_wait(range_word, SCALED_THREADS), a.x_absmax ? 14 : 8); };
        // `first`: the first block of this CTA, whose filter copy first_filter has issued
        auto open_stage = [&](const float* wt_tile, int kb, bool first) -> float* {
            const int k = st_k;
            if (k == 0) {
                const int s = st_idx;
                stage_A = stage0 + (long long)s * stage_floats;
                // use number u of this stage waits for the MMAs of use u-1; the first use passes at once
                if (!TDC_PROF_WAIT(0, mbar_wait(&empty_bar[s], (uint32_t)(st_use ^ 1)))) { *abort_flag = 1; return nullptr; }
                if (tid == 0 && !first) {
                    const uint32_t bytes = (uint32_t)(a.nkb - kb < a.kps ? a.nkb - kb : a.kps) * b_bytes;
                    mbar_expect_tx(&full_bar[s], bytes);
                    bulk_g2s(stage_A + a.kps * a_floats, wt_tile + (long long)kb * b_floats, bytes, &full_bar[s]);
                }
            }
            return stage_A + k * a_floats;
        };
        // after channel block kb is stored: the last block of a stage hands the stage over
        auto close_stage = [&](int kb) {
            if (++st_k == a.kps || kb == a.nkb - 1) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&full_bar[st_idx])) : "memory");
                st_k = 0;
                if (++st_idx == a.ns) { st_idx = 0; st_use ^= 1; }
            }
        };
        if constexpr (LD == LD_VEC) {
            auto put = [&](float* A, int q, int pp, float c0, float c1, float c2, float c3) {
                float4 hi;
                hi.x = to_tf32(c0); hi.y = to_tf32(c1); hi.z = to_tf32(c2); hi.w = to_tf32(c3);
                *reinterpret_cast<float4*>(A + ((q * a.P + pp) << 2)) = hi;
                if (a.hl == 2)
                    *reinterpret_cast<float4*>(A + CB * a.P + ((q * a.P + pp) << 2)) = make_float4(c0 - hi.x, c1 - hi.y, c2 - hi.z, c3 - hi.w);
            };
            // 1x1 filter, H*W a multiple of 4: a thread owns 4 consecutive positions x 4 channels of a block;
            // four 16-byte loads (one per channel), transposed in registers into four 16-byte stores
            for (long long t = blockIdx.x; t < ntiles && !*abort_flag; t += gridDim.x) {
                long long g0;
                int cnt, ocb;
                tile_of<MT>(a, t, g0, cnt, ocb);
                const int rows = cnt * M_TILE;                           // a one-tap filter has no halo
                const float* wt_tile = a.wt + (long long)ocb * a.nkb * b_floats;
                if (t == blockIdx.x) first_filter(wt_tile);
                bool ok = true;
                constexpr int NI = (MT * M_TILE / 2 + P_LOADERS - 1) / P_LOADERS;
                long long off[NI];
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    const int quad = (tid + i * P_LOADERS) >> 1;
                    off[i] = -1;
                    if (quad * 4 < rows) {
                        const long long g = g0 + quad * 4;
                        if (g < a.total_pos) { const long long b = image_of(a, g); off[i] = b * a.C * HW + (g - b * a.Lp); }
                    }
                }
                float4 va[NI][4], vb[NI][4];
                auto load = [&](int kb, float4 (&v)[NI][4]) {
#pragma unroll
                    for (int i = 0; i < NI; ++i) {
                        const int c0 = kb * CB + ((tid + i * P_LOADERS) & 1) * 4;
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            v[i][j] = (off[i] >= 0 && c0 + j < a.C) ? __ldg(reinterpret_cast<const float4*>(a.x + off[i] + (long long)(c0 + j) * HW))
                                                                     : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                };
                auto stage = [&](int kb, float4 (&v)[NI][4]) -> bool {
                    float* A = open_stage(wt_tile, kb, t == blockIdx.x && kb == 0);
                    if (!A) return false;
#pragma unroll
                    for (int i = 0; i < NI; ++i) {
                        const int item = tid + i * P_LOADERS, q = item & 1, pp = (item >> 1) * 4;
                        if (pp < rows) {
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
                for (int kb = 0; kb < a.nkb && ok; kb += 2) {
                    ok = stage(kb, va);
                    if (ok && kb + 2 < a.nkb) load(kb + 2, va);
                    if (ok && kb + 1 < a.nkb) {
                        ok = stage(kb + 1, vb);
                        if (ok && kb + 3 < a.nkb) load(kb + 3, vb);
                    }
                }
                if (!ok) break;
            }
        } else if constexpr (LD == LD_BULK) {
            // The raw slots are filled by the producer (below); these warps wait for a slot, pick their patch rows
            // out of its boxes, split them and store the operand layout, then hand the slot back.
            const float* raw0 = stage0 + (long long)a.ns * stage_floats;
            const int slot_floats = a.nbox_cap * (BOXC * BOXW), depth = a.depth;
            int r_slot = 0, r_use = 0;
            long long t = blockIdx.x;
            for (; t < ntiles && !*abort_flag; t += gridDim.x) {
                long long g0;
                int cnt, ocb;
                tile_of<MT>(a, t, g0, cnt, ocb);
                const int rows = cnt * M_TILE + halo_rows;
                const long long gp0 = g0 - a.shift;
                const float* wt_tile = a.wt + (long long)ocb * a.nkb * b_floats;
                if (t == blockIdx.x) first_filter(wt_tile);
                // offset of channel 0 of each owned patch row within a raw slot, -1 = a row of zeros
                int roff[PPT];
                TDC_PROF_SPAN_BEGIN;
                {
                    // Division-free but for the first row: a thread's rows are 256 positions apart, so (image, row,
                    // column) of the next one follow from the previous by adding (step_y, step_x) with carries.  The
                    // first position is taken one image up (gp0 may be negative by less than an image), image -1 = before x.
                    const int Hp = a.Hp;                                         // rows of a padded image
                    const long long g_first = gp0 + tid + a.Lp;
                    long long bi = image_of(a, g_first);
                    int rem = (int)(g_first - bi * a.Lp);
                    int yy = row_of(a, rem), xx = rem - yy * a.Wp;
                    bi -= 1;
                    // the runs of the images this patch meets, one image per lane: first pixel (rounded down to 16 bytes),
                    // boxes, and by a prefix sum the first box of each image in the raw slot
                    const long long lo = gp0 < 0 ? 0 : gp0, hi = (gp0 + rows < a.total_pos ? gp0 + rows : a.total_pos) - 1;
                    const long long b_first = image_of(a, lo), b_last = image_of(a, hi);
                    int my_pix4 = 0, my_nbox = 0;
                    if (b_first + lane <= b_last) image_run(a, gp0, rows, b_first + lane, my_pix4, my_nbox);
                    int my_box0 = my_nbox;                                       // inclusive scan, made exclusive below
#pragma unroll
                    for (int d = 1; d < 32; d <<= 1) {
                        const int v = __shfl_up_sync(0xffffffffu, my_box0, d);
                        if (lane >= d) my_box0 += v;
                    }
                    my_box0 -= my_nbox;
#pragma unroll
                    for (int i = 0; i < PPT; ++i) {
                        const int pp = tid + i * P_LOADERS;
                        const long long j = bi - b_first;                        // lane that holds this row's image
                        const int src = (j >= 0 && j < 32) ? (int)j : 0;
                        const int pix4 = __shfl_sync(0xffffffffu, my_pix4, src), box0 = __shfl_sync(0xffffffffu, my_box0, src);
                        roff[i] = -1;
                        if (pp < rows && bi >= 0 && bi < a.B && yy < a.H && xx < a.W && j >= 0 && j < 32) {
                            const int d = yy * a.W + xx - pix4;
                            roff[i] = (box0 + d / BOXW) * (BOXC * BOXW) + (d & (BOXW - 1));
                        }
                        xx += a.step_x; yy += a.step_y;                          // 256 positions on
                        if (xx >= a.Wp) { xx -= a.Wp; ++yy; }
                        while (yy >= Hp) { yy -= Hp; ++bi; }
                    }
                }
                TDC_PROF_SPAN_END(6);
                TDC_PROF_MARK(22, tid == 32, true);
                if (t == blockIdx.x) scale_here();                               // the range's round trip ran under the index work
                bool ok = true;
                for (int kb = 0; kb < a.nkb; ++kb) {
                    float* A = open_stage(wt_tile, kb, t == blockIdx.x && kb == 0);
                    if (!A || !TDC_PROF_WAIT(1, mbar_wait(&rfull_bar[r_slot], (uint32_t)r_use))) { *abort_flag = 1; ok = false; break; }
                    const float* R = raw0 + (long long)r_slot * slot_floats;
                    TDC_PROF_MARK(23, tid == 64, true);
                    TDC_PROF_SPAN_BEGIN;
#pragma unroll
                    for (int i = 0; i < PPT; ++i) {
                        const int pp = tid + i * P_LOADERS;
                        if (pp < rows) {
                            float c[CBK];
#pragma unroll
                            for (int j = 0; j < CBK; ++j) c[j] = roff[i] >= 0 ? R[roff[i] + j * BOXW] : 0.f;
                            store_row<F16>(A, a.P, a.hl, pp, c, xs);
                        }
                    }
                    TDC_PROF_SPAN_END(8);
                    __syncwarp();                                          // every lane has its values in registers
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&rempty_bar[r_slot])) : "memory");
                    if (++r_slot == depth) { r_slot = 0; r_use ^= 1; }
                    { TDC_PROF_SPAN_BEGIN; close_stage(kb); TDC_PROF_SPAN_END(9); }
                }
                if (!ok) { t = -1; break; }
            }
            if (t == blockIdx.x) scale_here();             // no tile was started: the draining warps still wait at the barrier
        } else {
            // The input goes global -> (cp.async, 4 bytes, zero-filled where the patch is padding) -> a ring of
            // raw fp32 slots in shared memory -> registers -> hi/lo split -> operand layout.  A thread copies and
            // later converts the SAME patch rows, so the ring needs no barrier, only cp.async.wait_group; it runs
            // `depth` channel blocks ahead and straight across tile boundaries, which keeps enough bytes in
            // flight to cover the memory latency and leaves no cold start at the beginning of a tile.
            float* raw0 = stage0 + (long long)a.ns * stage_floats;
            const int raw_floats = CBK * a.P, depth = a.depth;
            const long long my_tiles = blockIdx.x >= ntiles ? 0 : a.small ? (long long)((uint32_t)(ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x)
                                                                            : (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x;
            const long long total = my_tiles * a.nkb;
            long long src_off[PPT];              // of the tile being copied: offset of channel 0 of each owned row, -1 = zeros
            long long l_tile = blockIdx.x;       // copy side: tile, channel block and raw slot of the next block to issue
            int l_kb = 0, l_slot = 0, l_rows = 0, c_rows = 0;   // rows of the tile being copied / converted
            // gathering plans (TAPS != 9): a "channel" is an (input channel, filter row, filter column) triple — or, in the
            // strided-row plan, an (input channel, filter row, column phase) triple, the rest of the filter's columns
            // being taps — and a patch row is an output position, whose window starts at input (iy0, ix0), possibly outside
            const float* rbase[PPT];             // x at (image, channel 0, iy0, ix0) of each owned row (only formed, never read, when outside)
            int rmask[PPT];                      // bit dy: input row iy0 + dy exists; bit 16 + dx: input column ix0 + dx exists; 0 = no such position
            int g_ci = 0, g_dy = 0, g_dx = 0;    // the triple of the next channel to copy
            const int g_cin = (TAPS != 9 && a.gather) ? a.C / (a.gR * a.gS) : 0;
            auto issue = [&](long long li) {
                if (li < total) {
                    if (TAPS != 9 && a.gather) {
                        if (l_kb == 0) {
                            long long g0;
                            int cnt, ocb;
                            tile_of<MT>(a, l_tile, g0, cnt, ocb);
                            l_rows = cnt * M_TILE + halo_rows;
#pragma unroll
                            for (int i = 0; i < PPT; ++i) {
                                const int pp = tid + i * P_LOADERS;
                                rmask[i] = 0; rbase[i] = a.x;
                                const long long g = g0 - a.shift + pp;               // a plan with a phase starts one position early
                                if (pp < l_rows && g >= 0 && g < a.total_pos) {
                                    const long long b = image_of(a, g);
                                    const int rem = (int)(g - b * a.Lp);
                                    const int oy = row_of(a, rem), ox = rem - oy * a.Wp;
                                    const int iy0 = oy * a.stride - a.gpad, ix0 = ox * a.stride - a.gpadx;
                                    int m = 0;
                                    for (int d = 0; d < a.gR; ++d) m |= ((unsigned)(iy0 + d) < (unsigned)a.Hin) << d;
                                    for (int d = 0; d < a.gS; ++d) m |= ((unsigned)(ix0 + d) < (unsigned)a.Win) << (16 + d);
                                    rmask[i] = m;
                                    rbase[i] = a.x + (b * g_cin * a.HWin + (long long)iy0 * a.Win + ix0);
                                }
                            }
                            g_ci = g_dy = g_dx = 0;
                        }
                        if (a.gpair) {
                            // stride 2: the two column phases of a (channel, filter row) are neighbours in memory, on an even
                            // element: one 8-byte copy per pair; the raw slot holds [pair][patch row][2]
                            const uint32_t dst0 = smem_u32(raw0 + l_slot * raw_floats) + (uint32_t)tid * 8u;
#pragma unroll
                            for (int jp = 0; jp < CBK / 2; ++jp) {
                                const int delta = g_ci * (int)a.HWin + g_dy * a.Win;
                                const int sel = g_ci < g_cin ? ((1 << g_dy) | 0x10000) : -1;
#pragma unroll
                                for (int i = 0; i < PPT; ++i) {
                                    if (tid + i * P_LOADERS < l_rows) {
                                        const bool real = (rmask[i] & sel) == sel;
                                        const float* src = real ? rbase[i] + delta : a.x;
                                        asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;"
                                                     ::"r"(dst0 + (uint32_t)((jp * a.P + i * P_LOADERS) * 8)), "l"(src), "r"(real ? 8u : 0u) : "memory");
                                    }
                                }
                                if (++g_dy == a.gR) { g_dy = 0; ++g_ci; }
                            }
                        } else {
                        const uint32_t dst0 = smem_u32(raw0 + l_slot * raw_floats) + (uint32_t)tid * 4u;
#pragma unroll
                        for (int j = 0; j < CBK; ++j) {
                            const int delta = g_ci * (int)a.HWin + g_dy * a.Win + g_dx;     // the host keeps channels x image below 2^31
                            const int sel = g_ci < g_cin ? ((1 << g_dy) | (0x10000 << g_dx)) : -1;   // -1 never matches a mask
#pragma unroll
                            for (int i = 0; i < PPT; ++i) {
                                if (tid + i * P_LOADERS < l_rows) {
                                    const bool real = (rmask[i] & sel) == sel;
                                    const float* src = real ? rbase[i] + delta : a.x;
                                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;"
                                                 ::"r"(dst0 + (uint32_t)((j * a.P + i * P_LOADERS) * 4)), "l"(src), "r"(real ? 4u : 0u) : "memory");
                                }
                            }
                            if (++g_dx == a.gS) { g_dx = 0; if (++g_dy == a.gR) { g_dy = 0; ++g_ci; } }
                        }
                        }
                    } else {
                        if (l_kb == 0) {
                            long long g0;
                            int cnt, ocb;
                            tile_of<MT>(a, l_tile, g0, cnt, ocb);
                            l_rows = cnt * M_TILE + halo_rows;
                            const long long gp0 = g0 - a.shift;
#pragma unroll
                            for (int i = 0; i < PPT; ++i) {
                                const int pp = tid + i * P_LOADERS;
                                src_off[i] = -1;
                                if (pp < l_rows) {
                                    const long long g = gp0 + pp;
                                    if (g >= 0 && g < a.total_pos) {
                                        const long long b = image_of(a, g);
                                        const int rem = (int)(g - b * a.Lp);
                                        const int yy = row_of(a, rem), xx = rem - yy * a.Wp;
                                        if (yy < a.H && xx < a.W) src_off[i] = b * a.C * a.HWin + (long long)(yy * a.stride) * a.Win + xx * a.stride;
                                    }
                                }
                            }
                        }
                        float* R = raw0 + l_slot * raw_floats;
                        const int c0 = l_kb * CBK;
#pragma unroll
                        for (int i = 0; i < PPT; ++i) {
                            const int pp = tid + i * P_LOADERS;
                            if (pp < l_rows) {
                                const float* src = a.x + (src_off[i] >= 0 ? src_off[i] + (long long)c0 * a.HWin : 0);
#pragma unroll
                                for (int j = 0; j < CBK; ++j) {
                                    const bool real = src_off[i] >= 0 && c0 + j < a.C;
                                    cp_async4(R + j * a.P + pp, real ? src + (long long)j * a.HWin : a.x, real);
                                }
                            }
                        }
                    }
                    if (++l_kb == a.nkb) { l_kb = 0; l_tile += gridDim.x; }
                    if (++l_slot == depth) l_slot = 0;
                }
                asm volatile("cp.async.commit_group;" ::: "memory");      // an empty group past the end keeps the count uniform
            };
            if (total > 0) {
                long long g0_first;
                int cnt_first, ocb_first;
                tile_of<MT>(a, blockIdx.x, g0_first, cnt_first, ocb_first);
                first_filter(a.wt + (long long)ocb_first * a.nkb * b_floats);
            }
            for (int d = 0; d < depth; ++d) issue(d);
            TDC_PROF_MARK(22, tid == 32, true);
            scale_here();                                  // the range's round trip ran under the index work and the first copies
            long long c_tile = blockIdx.x;
            int c_kb = 0, c_slot = 0;
            const float* wt_tile = a.wt;
            auto enter_tile = [&]() {                      // convert side: rows and filter block of tile c_tile
                long long g0;
                int cnt, ocb;
                tile_of<MT>(a, c_tile, g0, cnt, ocb);
                c_rows = cnt * M_TILE + halo_rows;
                wt_tile = a.wt + (long long)ocb * a.nkb * b_floats;
            };
            if (total > 0) enter_tile();
            for (long long ci = 0; ci < total && !*abort_flag; ++ci) {
                float* A = open_stage(wt_tile, c_kb, ci == 0);
                if (!A) break;
                { TDC_PROF_SPAN_BEGIN; cp_async_wait_pending(depth - 1); TDC_PROF_SPAN_END(1); }   // block ci has landed (this thread's part)
                TDC_PROF_MARK(23, tid == 64, true);
                const float* R = raw0 + c_slot * raw_floats;
                if (++c_slot == depth) c_slot = 0;
#pragma unroll
                for (int i = 0; i < PPT; ++i) {
                    const int pp = tid + i * P_LOADERS;
                    if (pp < c_rows) {
                        float c[CBK];
                        if (TAPS != 9 && a.gpair) {
#pragma unroll
                            for (int jp = 0; jp < CBK / 2; ++jp) {
                                const float2 v = reinterpret_cast<const float2*>(R)[jp * a.P + pp];
                                c[2 * jp] = v.x; c[2 * jp + 1] = v.y;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < CBK; ++j) c[j] = R[j * a.P + pp];
                        }
                        store_row<F16>(A, a.P, a.hl, pp, c, xs);
                    }
                }
                close_stage(c_kb);
                issue(ci + depth);                                         // the slot just read is free again
                if (++c_kb == a.nkb) { c_kb = 0; c_tile += gridDim.x; if (ci + 1 < total) enter_tile(); }
            }
            asm volatile("cp.async.wait_all;" ::: "memory");
        }
    }
    if (warp < P_IW0) TDC_PROF_FLUSH(0);
    if (warp < P_IW0) {}
    else if (LD == LD_BULK && warp == P_PRODUCER) {
      {
        // ================= producer of the bulk loader: one thread =================
        // Per tile the list of boxes (first pixel, image) is the same for every channel block; a block's boxes go
        // to one raw slot, whose mbarrier counts their bytes (a box is written whole, padding included).
        if (lane == 0) {
            float* raw0 = stage0 + (long long)a.ns * stage_floats;
            const int slot_floats = a.nbox_cap * (BOXC * BOXW), depth = a.depth;
            int p_slot = 0, p_use = 0;
            for (long long t = blockIdx.x; t < ntiles && !*abort_flag; t += gridDim.x) {
                long long g0;
                int cnt, ocb;
                tile_of<MT>(a, t, g0, cnt, ocb);
                const int rows = cnt * M_TILE + halo_rows;
                const long long gp0 = g0 - a.shift;
                const long long lo = gp0 < 0 ? 0 : gp0, hi = (gp0 + rows < a.total_pos ? gp0 + rows : a.total_pos) - 1;
                int nb = 0;
                for (long long b = image_of(a, lo), b_last = image_of(a, hi); b <= b_last; ++b) {
                    int pix4, nbox;
                    image_run(a, gp0, rows, b, pix4, nbox);
                    for (int k = 0; k < nbox; ++k, ++nb)
                        if (nb < a.nbox_cap) box_tab[nb] = make_int2(pix4 + k * BOXW, (int)b);
                }
                if (nb > a.nbox_cap) { *abort_flag = 1; break; }      // the host sized the slots for fewer boxes: give up rather than drop pixels
                bool ok = true;
                for (int kb = 0; kb < a.nkb; ++kb) {
                    if (!TDC_PROF_WAIT(2, mbar_wait(&rempty_bar[p_slot], (uint32_t)(p_use ^ 1)))) { *abort_flag = 1; ok = false; break; }
                    float* dst = raw0 + (long long)p_slot * slot_floats;
                    mbar_expect_tx(&rfull_bar[p_slot], (uint32_t)nb * (uint32_t)(BOXC * BOXW * 4));
                    for (int i = 0; i < nb; ++i) {
                        const int2 bx = box_tab[i];
                        bulk_tensor_3d(dst + i * (BOXC * BOXW), &tmap, bx.x, kb * BOXC, bx.y, &rfull_bar[p_slot]);
                        TDC_PROF_MARK(21, true, true);
                    }
                    if (++p_slot == depth) { p_slot = 0; p_use ^= 1; }
                }
                if (!ok) break;
            }
            // leaving early (another role gave up): no copy of this CTA may still be in flight when it exits, so
            // wait (bounded) for the last copies issued into every slot; slots never used pass at once
            if (*abort_flag)
                for (int d = 0; d < depth; ++d) mbar_wait(&rfull_bar[d], (uint32_t)(d < p_slot ? p_use : p_use ^ 1));
            TDC_PROF_FLUSH(1);
        }
        __syncwarp();
      }
    }
    else if (warp < P_EW0) {
        // ================= MMA issuers: warp P_IW0 + mt owns position tile mt =================
        const int mt = __shfl_sync(0xffffffffu, warp - P_IW0, 0);
        if (mt < MT) {
            long long j = 0;                    // accumulator hand-overs so far: one per tile and run
            int st_idx = 0, st_use = 0;         // stage to consume next, parity of its use count
            for (long long t = blockIdx.x; t < ntiles && !*abort_flag; t += gridDim.x) {
                long long g0_unused;
                int cnt, ocb_unused;
                tile_of<MT>(a, t, g0_unused, cnt, ocb_unused);
                if (mt >= cnt) {
                    // a smaller tile of the last round (always a CTA's last tile) has no position tile for this warp:
                    // it only keeps the stages' hand-over in step, one arrival per stage use
                    bool fine = true;
                    for (int kb0 = 0; kb0 < a.nkb && fine; kb0 += a.kps) {
                        fine = mbar_wait(&full_bar[st_idx], (uint32_t)st_use);
                        if (fine && lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&empty_bar[st_idx])) : "memory");
                        if (++st_idx == a.ns) { st_idx = 0; st_use ^= 1; }
                    }
                    if (!fine) { *abort_flag = 1; break; }
                    j += a.nseg;
                    continue;
                }
                bool ok = true;
                for (int seg = 0; seg < a.nseg && ok; ++seg, ++j) {
                    const int slot = (nbuf == 2 ? (int)(j & 1) : 0) * MT + mt;       // nbuf is 1 or 2
                    const int kb_lo = seg * a.seg_blocks, kb_hi = kb_lo + a.seg_blocks < a.nkb ? kb_lo + a.seg_blocks : a.nkb;
                    // the epilogue must have emptied this accumulator slot (its previous use); the first use passes at once
                    if (!TDC_PROF_WAIT(3, mbar_wait(&tempty_bar[slot], (uint32_t)((((nbuf == 2 ? j >> 1 : j)) & 1) ^ 1)))) { *abort_flag = 1; ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t d_main = tmem + (uint32_t)(slot * a.tile_cols);
                    for (int kb0 = kb_lo; kb0 < kb_hi; kb0 += a.kps) {
                        const int s = st_idx;
                        if (!TDC_PROF_WAIT(4, mbar_wait(&full_bar[s], (uint32_t)st_use))) { *abort_flag = 1; ok = false; break; }
                        if (++st_idx == a.ns) { st_idx = 0; st_use ^= 1; }
                        TDC_PROF_MARK(17, mt == 0 && lane == 0, true);
                        TDC_PROF_ISSUE_BEGIN;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const float* A = stage0 + (long long)s * stage_floats;
                        const int kend = kb0 + a.kps < kb_hi ? kb0 + a.kps : kb_hi;
                        if (elect_one()) {
                            for (int kb = kb0; kb < kend; ++kb) {
                                const int kr = kb - kb_lo;                    // block of this run
                                issue_block<NT, TAPS, F16>(a, d_main, smem_u32(A + (kb - kb0) * a_floats), smem_u32(A + a.kps * a_floats + (kb - kb0) * b_floats),
                                                           (uint32_t)(mt * M_TILE), kr & 1, kr < 2 && (kr == 0 || a.nmain == 2));
                            }
                            mma_commit(&empty_bar[s]);                        // the stage may be refilled when these MMAs are done
                            if (kend == kb_hi) mma_commit(&tfull_bar[slot]);  // and this run's accumulators are complete
                        }
                        __syncwarp();
                        TDC_PROF_ISSUE_END;
                    }
                }
                if (!ok) break;
            }
            TDC_PROF_MARK(18, mt == 0 && lane == 0, false);
            TDC_PROF_FLUSH(2);
        }
    } else {
        // ================= epilogue: P_GROUPS groups of four warps (one lane quarter of tensor memory per warp).
        // The work items of a CTA tile are (position tile, chunk of P_EPI_W channels) pairs, dealt to the groups in turn: the
        // epilogue is a latency chain (tensor memory -> registers -> residual loads -> stores), and several chains in
        // flight hide more of it than one; all groups start on the first position tile, whose issuer is released first.
        const int grp = (warp - P_EW0) >> 2;       // warps P_EW0 .. P_EW0 + 4 * P_GROUPS - 1
        // fp16 operands: the range of the input (its given partial maxima of |x|, or samples of x when there is no bound)
        // is loaded by these warps, which have nothing else to do yet and no registers in use; the round trip runs under
        // the index work of the loaders' first tile, which meet them at the barrier when that is done.
        if constexpr (F16) {
            unsigned int range_raw[RANGE_PER_THREAD];
            range_load(a.x_absmax, a.x, a.x_count, tid - P_EW0 * 32, 128 * P_GROUPS, range_raw);
            xs = range_scale(range_max(range_raw, range_word, SCALED_THREADS), a.x_absmax ? 14 : 8);
            inv = 1.f / (xs * a.w_scale[0]);
        }
        const int q = warp & 3;
        constexpr int CHUNKS = NT / P_EPI_W;
        long long j = 0;
        float ymax = 0.f;                       // largest magnitude this thread stored, compared as a bit pattern (so a NaN counts as large)
        float* const track = (F16 || a.y_absmax) ? &ymax : nullptr;
        for (long long t = blockIdx.x; t < ntiles && !*abort_flag; t += gridDim.x) {
            long long g0;
            int cnt, ocb;
            tile_of<MT>(a, t, g0, cnt, ocb);
            bool ok = true;
            for (int seg = 0; seg < a.nseg && ok; ++seg, ++j) {
                const int kb_lo = seg * a.seg_blocks, blocks = (kb_lo + a.seg_blocks < a.nkb ? kb_lo + a.seg_blocks : a.nkb) - kb_lo;
#pragma unroll 1
                for (int item = grp; item < cnt * CHUNKS && ok; item += P_GROUPS) {
                    const int mt = item / CHUNKS, chunk = item - mt * CHUNKS;
                    // the position tiles of a CTA tile are handed over one by one: while this one is drained, the
                    // issuers of the others still run, and its own issuer may start on the next run or CTA tile
                    const int slot = (nbuf == 2 ? (int)(j & 1) : 0) * MT + mt;
                    if (!TDC_PROF_WAIT(5, mbar_wait(&tfull_bar[slot], (uint32_t)((nbuf == 2 ? j >> 1 : j) & 1)))) { *abort_flag = 1; ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const long long g = g0 + mt * M_TILE + q * 32 + lane;
                    long long out_off = -1;
                    if (g < a.total_pos) {
                        const long long b = image_of(a, g);
                        const int rem = (int)(g - b * a.Lp);
                        const int yy = row_of(a, rem), xx = rem - yy * a.Wp;
                        if (yy < a.H && xx < a.W) out_off = b * a.K * HW + (long long)yy * a.W + xx;
                    }
                    uint32_t r[P_EPI_W];
                    load_chunk<NT, F16, P_EPI_W>(a, tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(slot * a.tile_cols + chunk * P_EPI_W), r, blocks, inv);
                    // this chunk of the slot is in registers: one arrival per warp and chunk hands the slot back when
                    // all of its chunks have been read, before the stores
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&tempty_bar[slot])) : "memory");
                    { TDC_PROF_SPAN_BEGIN;
                      store_chunk<P_EPI_W>(a, r, out_off, ocb * NT + chunk * P_EPI_W, HW, seg > 0, seg == a.nseg - 1, seg == a.nseg - 1 ? track : nullptr);
                      TDC_PROF_SPAN_END(7); }
                }
            }
            if (!ok) break;
        }
        if (track) {
            const unsigned int m = __reduce_max_sync(0xffffffffu, __float_as_uint(ymax));
            if (lane == 0) atomicMax(max_word, m);
        }
        TDC_PROF_FLUSH(3);
    }

    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    TDC_PROF_MARK(19, tid == 0, false);
    TDC_PROF_COUNT(20, tid == 0);
    if (*abort_flag && tid == 0 && a.status) atomicCAS(a.status, 0, 1);
    // an output that is not finite: the input went beyond fp16's range even after scaling (or was not finite itself)
    if (F16 && tid == 0 && a.status && *max_word >= 0x7f800000u) atomicCAS(a.status, 0, 2);
    if (a.y_absmax) {                           // entry = CTA; CTA 0 clears the entries no CTA owns
        if (tid == 0) a.y_absmax[blockIdx.x] = __uint_as_float(*max_word);
        if (blockIdx.x == 0)
            for (int i = gridDim.x + tid; i < ABSMAX_SLOTS; i += P_THREADS) a.y_absmax[i] = 0.f;
    }
    if (warp == P_IW0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)a.tmem_cols) : "memory");
}

}  // namespace tdc_tc
