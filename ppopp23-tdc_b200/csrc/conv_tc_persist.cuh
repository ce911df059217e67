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
//   * two groups of four epilogue warps (12-15, 16-19) take the (position tile, 32-channel chunk)
//     items of a CTA tile in turn; an accumulator is handed back as soon as all its chunks are in
//     registers, before the stores.
// Every mbarrier wait is bounded; a wait that runs out raises the CTA's abort flag, every
// role leaves its loop at the next check, the status word is set and tensor memory is freed.
#pragma once

namespace tdc_tc {

#ifndef TDC_TC_EPI_GROUPS
#define TDC_TC_EPI_GROUPS 2
#endif
constexpr int P_GROUPS  = TDC_TC_EPI_GROUPS;          // groups of four epilogue warps
constexpr int P_THREADS = 384 + 128 * P_GROUPS;     // 8 loader warps, 4 issuer warps (one lane each), the epilogue groups
constexpr int P_HEADER  = 256;   // bytes of barriers and flags in front of the stages

// Tile t of the list -> first output position, position tiles it holds (`cnt` <= MT), output-channel block.
// Tiles of the complete rounds hold MT position tiles; what is left for the last, partial round is spread over
// all CTAs as smaller tiles (with one output-channel block; a.full_groups covers every tile otherwise), so the
// launch ends after a part of a round instead of a whole one.
template <int MT>
__device__ __forceinline__ void tile_of(const Args& a, long long t, long long& g0, int& cnt, int& ocb) {
    long long tg = t;
    ocb = 0;
    if (a.n_ocb > 1) { tg = t / a.n_ocb; ocb = (int)(t - tg * a.n_ocb); }
    if (tg < a.full_groups) { g0 = tg * (MT * M_TILE); cnt = MT; return; }
    const long long first = a.tail_first_pt + (tg - a.full_groups) * a.tail_cnt, left = a.pt_total - first;
    g0 = first * M_TILE;
    cnt = left < a.tail_cnt ? (int)left : a.tail_cnt;
}

template <int NT, int MT, int TAPS, bool VEC>
__global__ void __launch_bounds__(P_THREADS) conv_tc_persist_kernel(const Args a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    uint64_t* full_bar   = reinterpret_cast<uint64_t*>(smem_raw);    // [ns]  patch stored + filter landed
    uint64_t* empty_bar  = full_bar + 4;                              // [ns]  MMAs that read the stage are done
    uint64_t* tfull_bar  = empty_bar + 4;                             // [nbuf*MT] the accumulators of a 128-position tile are complete
    uint64_t* tempty_bar = tfull_bar + 8;                             // [nbuf*MT] the epilogue has read them
    uint32_t* tmem_slot  = reinterpret_cast<uint32_t*>(tempty_bar + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float*    stage0     = reinterpret_cast<float*>(smem_raw + P_HEADER);

    // patch rows per loader thread: MT x 128 positions, plus two image rows of halo for a 3x3 filter (the host keeps
    // the patch within PPT x 256 rows; images up to 256 wide)
    constexpr int PPT = TAPS == 1 ? (MT >= 2 ? MT / 2 : 1) : (MT == 1 ? 3 : 4);
    // a stage holds a.kps channel blocks (one for 3x3 filters; several for one-tap filters, whose stages would
    // otherwise be all hand-over and no work): [kps input blocks][kps filter blocks]
    const int a_floats = a.hl * CB * a.P, b_floats = a.hl * TAPS * CB * NT, stage_floats = a.kps * (a_floats + b_floats);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int pad = (a.taps_r - 1) / 2;
    const int halo_rows = 2 * pad * (a.Wp + 1);                  // patch rows beyond the positions of a tile
    const long long HW = (long long)a.H * a.W;
    const uint32_t b_bytes = (uint32_t)b_floats * 4u;
    const int nbuf = a.nbuf;
    const long long ntiles = a.ntiles;          // position tiles x output-channel blocks

    if (tid == 0) {
        for (int s = 0; s < a.ns; ++s) { mbar_init(&full_bar[s], LOADERS / 32 + 1); mbar_init(&empty_bar[s], MT); }   // one arrival per loader warp + the filter's bytes
        for (int b = 0; b < 8; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], 4 * (NT / 32)); }   // one per issuer; one per epilogue warp and 32-channel chunk
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)a.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    if (warp < 8) {
        // ================= loaders =================
        // no division in these loops: the loaders are bound by instruction latency (two warps per scheduler), so the
        // ring positions are counters that wrap, not quotients of a running index
        int st_idx = 0, st_use = 0, st_k = 0;    // stage being filled, parity of its use count, blocks stored in it
        float* stage_A = nullptr;                // the stage being filled
        // where channel block kb of the current tile goes; its first block of a stage waits for the stage and starts
        // the copy of the stage's filter blocks
        auto open_stage = [&](const float* wt_tile, int kb) -> float* {
            const int k = st_k;
            if (k == 0) {
                const int s = st_idx;
                stage_A = stage0 + (long long)s * stage_floats;
                // use number u of this stage waits for the MMAs of use u-1; the first use passes at once
                if (!mbar_wait(&empty_bar[s], (uint32_t)(st_use ^ 1))) { *abort_flag = 1; return nullptr; }
                if (tid == 0) {
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
        auto put = [&](float* A, int q, int pp, float c0, float c1, float c2, float c3) {
            float4 hi;
            hi.x = to_tf32(c0); hi.y = to_tf32(c1); hi.z = to_tf32(c2); hi.w = to_tf32(c3);
            *reinterpret_cast<float4*>(A + ((q * a.P + pp) << 2)) = hi;
            if (a.hl == 2)
                *reinterpret_cast<float4*>(A + CB * a.P + ((q * a.P + pp) << 2)) = make_float4(c0 - hi.x, c1 - hi.y, c2 - hi.z, c3 - hi.w);
        };
        if constexpr (VEC) {
            // 1x1 filter, H*W a multiple of 4: a thread owns 4 consecutive positions x 4 channels of a block;
            // four 16-byte loads (one per channel), transposed in registers into four 16-byte stores
            for (long long t = blockIdx.x; t < ntiles && !*abort_flag; t += gridDim.x) {
                long long g0;
                int cnt, ocb;
                tile_of<MT>(a, t, g0, cnt, ocb);
                const int rows = cnt * M_TILE;                           // a one-tap filter has no halo
                const float* wt_tile = a.wt + (long long)ocb * a.nkb * b_floats;
                bool ok = true;
                constexpr int NI = (MT * M_TILE / 2 + LOADERS - 1) / LOADERS;
                long long off[NI];
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    const int quad = (tid + i * LOADERS) >> 1;
                    off[i] = -1;
                    if (quad * 4 < rows) {
                        const long long g = g0 + quad * 4;
                        if (g < a.total_pos) { const long long b = g / a.Lp; off[i] = b * a.C * HW + (g - b * a.Lp); }
                    }
                }
                float4 va[NI][4], vb[NI][4];
                auto load = [&](int kb, float4 (&v)[NI][4]) {
#pragma unroll
                    for (int i = 0; i < NI; ++i) {
                        const int c0 = kb * CB + ((tid + i * LOADERS) & 1) * 4;
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            v[i][j] = (off[i] >= 0 && c0 + j < a.C) ? __ldg(reinterpret_cast<const float4*>(a.x + off[i] + (long long)(c0 + j) * HW))
                                                                     : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                };
                auto stage = [&](int kb, float4 (&v)[NI][4]) -> bool {
                    float* A = open_stage(wt_tile, kb);
                    if (!A) return false;
#pragma unroll
                    for (int i = 0; i < NI; ++i) {
                        const int item = tid + i * LOADERS, q = item & 1, pp = (item >> 1) * 4;
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
        } else {
            // The input goes global -> (cp.async, 4 bytes, zero-filled where the patch is padding) -> a ring of
            // raw fp32 slots in shared memory -> registers -> hi/lo split -> operand layout.  A thread copies and
            // later converts the SAME patch rows, so the ring needs no barrier, only cp.async.wait_group; it runs
            // `depth` channel blocks ahead and straight across tile boundaries, which keeps enough bytes in
            // flight to cover the memory latency and leaves no cold start at the beginning of a tile.
            float* raw0 = stage0 + (long long)a.ns * stage_floats;
            const int raw_floats = CB * a.P, depth = a.depth;
            const long long my_tiles = blockIdx.x < ntiles ? (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
            const long long total = my_tiles * a.nkb;
            long long src_off[PPT];              // of the tile being copied: offset of channel 0 of each owned row, -1 = zeros
            long long l_tile = blockIdx.x;       // copy side: tile, channel block and raw slot of the next block to issue
            int l_kb = 0, l_slot = 0, l_rows = 0, c_rows = 0;   // rows of the tile being copied / converted
            // general plan (TAPS == 1 only): a "channel" is an (input channel, filter row, filter column) triple
            // and a patch row is an output position, whose window starts at input (iy0, ix0), possibly outside
            const float* rbase[PPT];             // x at (image, channel 0, iy0, ix0) of each owned row (only formed, never read, when outside)
            int rmask[PPT];                      // bit dy: input row iy0 + dy exists; bit 16 + dx: input column ix0 + dx exists; 0 = no such position
            int g_ci = 0, g_dy = 0, g_dx = 0;    // the triple of the next channel to copy
            const int g_cin = (TAPS == 1 && a.gather) ? a.C / (a.gR * a.gS) : 0;
            auto issue = [&](long long li) {
                if (li < total) {
                    if (TAPS == 1 && a.gather) {
                        if (l_kb == 0) {
                            long long g0;
                            int cnt, ocb;
                            tile_of<MT>(a, l_tile, g0, cnt, ocb);
                            l_rows = cnt * M_TILE;
#pragma unroll
                            for (int i = 0; i < PPT; ++i) {
                                const int pp = tid + i * LOADERS;
                                rmask[i] = 0; rbase[i] = a.x;
                                const long long g = g0 + pp;
                                if (pp < l_rows && g < a.total_pos) {
                                    const long long b = g / a.Lp;
                                    const int rem = (int)(g - b * a.Lp);
                                    const int oy = rem / a.Wp, ox = rem - oy * a.Wp;
                                    const int iy0 = oy * a.stride - a.gpad, ix0 = ox * a.stride - a.gpad;
                                    int m = 0;
                                    for (int d = 0; d < a.gR; ++d) m |= ((unsigned)(iy0 + d) < (unsigned)a.Hin) << d;
                                    for (int d = 0; d < a.gS; ++d) m |= ((unsigned)(ix0 + d) < (unsigned)a.Win) << (16 + d);
                                    rmask[i] = m;
                                    rbase[i] = a.x + (b * g_cin * a.HWin + (long long)iy0 * a.Win + ix0);
                                }
                            }
                            g_ci = g_dy = g_dx = 0;
                        }
                        const uint32_t dst0 = smem_u32(raw0 + l_slot * raw_floats) + (uint32_t)tid * 4u;
#pragma unroll
                        for (int j = 0; j < CB; ++j) {
                            const int delta = g_ci * (int)a.HWin + g_dy * a.Win + g_dx;     // the host keeps channels x image below 2^31
                            const int sel = g_ci < g_cin ? ((1 << g_dy) | (0x10000 << g_dx)) : -1;   // -1 never matches a mask
#pragma unroll
                            for (int i = 0; i < PPT; ++i) {
                                if (tid + i * LOADERS < l_rows) {
                                    const bool real = (rmask[i] & sel) == sel;
                                    const float* src = real ? rbase[i] + delta : a.x;
                                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;"
                                                 ::"r"(dst0 + (uint32_t)((j * a.P + i * LOADERS) * 4)), "l"(src), "r"(real ? 4u : 0u) : "memory");
                                }
                            }
                            if (++g_dx == a.gS) { g_dx = 0; if (++g_dy == a.gR) { g_dy = 0; ++g_ci; } }
                        }
                    } else {
                        if (l_kb == 0) {
                            long long g0;
                            int cnt, ocb;
                            tile_of<MT>(a, l_tile, g0, cnt, ocb);
                            l_rows = cnt * M_TILE + halo_rows;
                            const long long gp0 = g0 - (long long)pad * (a.Wp + 1);
#pragma unroll
                            for (int i = 0; i < PPT; ++i) {
                                const int pp = tid + i * LOADERS;
                                src_off[i] = -1;
                                if (pp < l_rows) {
                                    const long long g = gp0 + pp;
                                    if (g >= 0 && g < a.total_pos) {
                                        const long long b = g / a.Lp;
                                        const int rem = (int)(g - b * a.Lp);
                                        const int yy = rem / a.Wp, xx = rem - yy * a.Wp;
                                        if (yy < a.H && xx < a.W) src_off[i] = b * a.C * a.HWin + (long long)(yy * a.stride) * a.Win + xx * a.stride;
                                    }
                                }
                            }
                        }
                        float* R = raw0 + l_slot * raw_floats;
                        const int c0 = l_kb * CB;
#pragma unroll
                        for (int i = 0; i < PPT; ++i) {
                            const int pp = tid + i * LOADERS;
                            if (pp < l_rows) {
                                const float* src = a.x + (src_off[i] >= 0 ? src_off[i] + (long long)c0 * a.HWin : 0);
#pragma unroll
                                for (int j = 0; j < CB; ++j) {
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
            for (int d = 0; d < depth; ++d) issue(d);
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
                float* A = open_stage(wt_tile, c_kb);
                if (!A) break;
                cp_async_wait_pending(depth - 1);                         // block ci has landed (this thread's part)
                const float* R = raw0 + c_slot * raw_floats;
                if (++c_slot == depth) c_slot = 0;
#pragma unroll
                for (int i = 0; i < PPT; ++i) {
                    const int pp = tid + i * LOADERS;
                    if (pp < c_rows) {
#pragma unroll
                        for (int q = 0; q < CB / 4; ++q)
                            put(A, q, pp, R[(4 * q) * a.P + pp], R[(4 * q + 1) * a.P + pp], R[(4 * q + 2) * a.P + pp], R[(4 * q + 3) * a.P + pp]);
                    }
                }
                close_stage(c_kb);
                issue(ci + depth);                                         // the slot just read is free again
                if (++c_kb == a.nkb) { c_kb = 0; c_tile += gridDim.x; if (ci + 1 < total) enter_tile(); }
            }
            asm volatile("cp.async.wait_all;" ::: "memory");
        }
    }
    else if (warp < 12) {
        // ================= MMA issuers: warp 8+mt owns position tile mt =================
        const int mt = __shfl_sync(0xffffffffu, warp - 8, 0);
        if (mt < MT) {
            long long j = 0;                    // tiles done by this CTA
            int st_idx = 0, st_use = 0;         // stage to consume next, parity of its use count
            for (long long t = blockIdx.x; t < ntiles && !*abort_flag; t += gridDim.x, ++j) {
                const int slot = (int)(j % nbuf) * MT + mt;
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
                    continue;
                }
                // the epilogue must have emptied this accumulator slot (its previous use); the first use passes at once
                if (!mbar_wait(&tempty_bar[slot], (uint32_t)(((j / nbuf) & 1) ^ 1))) { *abort_flag = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_main = tmem + (uint32_t)(slot * a.tile_cols);
                bool ok = true;
                for (int kb0 = 0; kb0 < a.nkb; kb0 += a.kps) {
                    const int s = st_idx;
                    if (!mbar_wait(&full_bar[s], (uint32_t)st_use)) { *abort_flag = 1; ok = false; break; }
                    if (++st_idx == a.ns) { st_idx = 0; st_use ^= 1; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const float* A = stage0 + (long long)s * stage_floats;
                    const int kend = kb0 + a.kps < a.nkb ? kb0 + a.kps : a.nkb;
                    if (elect_one()) {
                        for (int kb = kb0; kb < kend; ++kb)
                            issue_block<NT, TAPS>(a, d_main, smem_u32(A + (kb - kb0) * a_floats), smem_u32(A + a.kps * a_floats + (kb - kb0) * b_floats),
                                                  (uint32_t)(mt * M_TILE), kb & 1, kb < 2 && (kb == 0 || a.nmain == 2));
                        mma_commit(&empty_bar[s]);                        // the stage may be refilled when these MMAs are done
                        if (kend == a.nkb) mma_commit(&tfull_bar[slot]);  // and this position tile's accumulators are complete
                    }
                    __syncwarp();
                }
                if (!ok) break;
            }
        }
    } else {
        // ================= epilogue: P_GROUPS groups of four warps (one lane quarter of tensor memory per warp).
        // The work items of a CTA tile are (position tile, 32-channel chunk) pairs, dealt to the groups in turn: the
        // epilogue is a latency chain (tensor memory -> registers -> residual loads -> stores), and several chains in
        // flight hide more of it than one; all groups start on the first position tile, whose issuer is released first.
        const int grp = (warp - 12) >> 2;
        const int q = warp & 3;
        constexpr int CHUNKS = NT / 32;
        long long j = 0;
        for (long long t = blockIdx.x; t < ntiles && !*abort_flag; t += gridDim.x, ++j) {
            long long g0;
            int cnt, ocb;
            tile_of<MT>(a, t, g0, cnt, ocb);
            bool ok = true;
#pragma unroll 1
            for (int item = grp; item < cnt * CHUNKS && ok; item += P_GROUPS) {
                const int mt = item / CHUNKS, chunk = item - mt * CHUNKS;
                // the position tiles of a CTA tile are handed over one by one: while this one is drained, the
                // issuers of the others still run, and its own issuer may start on the next CTA tile
                const int slot = (int)(j % nbuf) * MT + mt;
                if (!mbar_wait(&tfull_bar[slot], (uint32_t)((j / nbuf) & 1))) { *abort_flag = 1; ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const long long g = g0 + mt * M_TILE + q * 32 + lane;
                long long out_off = -1;
                if (g < a.total_pos) {
                    const long long b = g / a.Lp;
                    const int rem = (int)(g - b * a.Lp);
                    const int yy = rem / a.Wp, xx = rem - yy * a.Wp;
                    if (yy < a.H && xx < a.W) out_off = b * a.K * HW + (long long)yy * a.W + xx;
                }
                uint32_t r[32];
                load_chunk<NT>(a, tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(slot * a.tile_cols + chunk * 32), r);
                // this chunk of the slot is in registers: one arrival per warp and chunk hands the slot back when
                // all of its chunks have been read, before the stores
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&tempty_bar[slot])) : "memory");
                store_chunk(a, r, out_off, ocb * NT + chunk * 32, HW);
            }
            if (!ok) break;
        }
    }

    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_flag && tid == 0 && a.status) atomicCAS(a.status, 0, 1);
    if (warp == 8) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)a.tmem_cols) : "memory");
}

}  // namespace tdc_tc
