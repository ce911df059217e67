// Tile geometry and the analytical tile selector (host code only).
//
// The reference picks TH/TW/TC either by exhaustive search over a measured table
// (A100-evaluation/TDC-LAYERS-ORACLE/gen_from_occupancy.py:51-66) or by an analytical
// model over the moved volumes and a flops*waves term
// (A100-evaluation/TDC-LAYERS-MODELING/model.py:135-234).  The model below keeps those
// terms but counts them for this kernel's CTA (several output channels per thread, all
// input channels walked by one CTA) and for B200's SM count, register file and shared
// memory, and it turns them into one cycle estimate instead of the reference's
// "keep the first 5% of the enumeration, then take the least input volume".
#include "tile.h"
#include <algorithm>
#include <cmath>
#include <vector>

namespace tdc {

static inline int cdiv(int a, int b) { return (a + b - 1) / b; }
static inline int rup(int a, int b) { return cdiv(a, b) * b; }

static void all_variants(std::vector<const Variant*>* out) {
    int n;
    const Variant* p;
    p = variants_3x3s1(&n); for (int i = 0; i < n; ++i) out->push_back(p + i);
    p = variants_3x3s2(&n); for (int i = 0; i < n; ++i) out->push_back(p + i);
    p = variants_1x1(&n);   for (int i = 0; i < n; ++i) out->push_back(p + i);
    p = variants_rt(&n);    for (int i = 0; i < n; ++i) out->push_back(p + i);
}

static const std::vector<const Variant*>& registry() {
    static std::vector<const Variant*> r = [] { std::vector<const Variant*> v; all_variants(&v); return v; }();
    return r;
}

static bool variant_fits(const Variant& v, const Shape& s, bool exact) {
    if (v.stride != s.stride) return false;
    if (exact) return v.kh == s.R && v.kw == s.S;
    return v.kh == 0 && s.R <= 7 && s.S <= 7;
}

const Variant* find_variant(const Shape& s, const tdc_tile& t) {
    for (int pass = 0; pass < 2; ++pass)
        for (const Variant* v : registry())
            if (variant_fits(*v, s, pass == 0) && v->tn == t.tn && v->th == t.th && v->tw == t.tw &&
                v->nog == t.nog)
                return v;
    return nullptr;
}

int make_geometry(const Shape& s, const tdc_tile& t, const tdc_devinfo& dev, Geometry* g, const char** why) {
    const char* dummy;
    if (!why) why = &dummy;
    if (t.th <= 0 || t.tw <= 0 || t.tc <= 0 || t.tn <= 0 || t.nog <= 0 || t.gy <= 0 || t.gx <= 0 ||
        t.imgs <= 0 || t.ks <= 0 || t.kc <= 0) { *why = "tile has a field <= 0"; return TDC_ERR_TILE; }
    const Variant* v = find_variant(s, t);
    if (!v) { *why = "no compiled kernel for this filter size / stride / (tn,th,tw,nog)"; return TDC_ERR_UNSUPPORTED; }
    const int Ho = s.Ho(), Wo = s.Wo();
    if (t.tc % t.ks) { *why = "tc must be a multiple of ks"; return TDC_ERR_TILE; }
    if (t.kc > 8) { *why = "kc (cluster size) must be 1..8"; return TDC_ERR_TILE; }
    if (t.imgs > 1 && (t.gy * t.th < Ho || t.gx * t.tw < Wo)) {
        *why = "imgs > 1 needs gy*th >= Ho and gx*tw >= Wo"; return TDC_ERR_TILE;
    }
    g->v = v;
    g->in_rows = (t.gy * t.th - 1) * s.stride + s.R;
    g->in_w    = (t.gx * t.tw - 1) * s.stride + s.S;
    // Row stride of the staged patch. Tiles whose row window is read with 16-byte loads need
    // a multiple of 4 words, and two thread rows that share a quarter-warp (nog < 8) must
    // not start on the same banks; tiles read word by word take the first stride for which
    // the pixel groups of a warp fall on distinct banks.
    const bool vec = (v->kh != 0) && ((t.tw * s.stride) % 4 == 0);
    if (vec) {
        g->in_wp = rup(g->in_w, 4);
        if (t.nog < 8) while ((t.th * s.stride * g->in_wp) % 32 == 0) g->in_wp += 4;
    } else {
        const int groups = std::max(1, 32 / t.nog);
        g->in_wp = g->in_w;
        for (int cand = g->in_w; cand < g->in_w + 16; ++cand) {
            unsigned seen = 0; bool clash = false;
            for (int pgi = 0; pgi < groups && pgi < t.gy * t.gx; ++pgi) {
                int bank = ((pgi % t.gx) * t.tw * s.stride + (pgi / t.gx) * t.th * s.stride * cand) & 31;
                if (seen & (1u << bank)) { clash = true; break; }
                seen |= 1u << bank;
            }
            if (!clash) { g->in_wp = cand; break; }
        }
    }
    g->patch   = rup(t.imgs * g->in_rows * g->in_wp, 4);
    g->tiles_y = cdiv(Ho, t.gy * t.th);
    g->tiles_x = cdiv(Wo, t.gx * t.tw);
    g->img_groups = cdiv(s.B, t.imgs);
    g->n_ocb   = cdiv(s.K, t.tn * t.nog);
    g->nt      = t.nog * t.imgs * t.gy * t.gx;
    g->threads = g->nt * t.ks;
    if (g->threads > v->maxt) { *why = "tile needs more threads per CTA than this thread tile allows"; return TDC_ERR_TILE; }
    if ((long long)t.imgs * s.C * s.H * s.W >= (1ll << 31)) { *why = "images of one CTA exceed 2^31 elements"; return TDC_ERR_TILE; }
    g->stage_floats = t.tc * g->patch + t.tc * s.R * s.S * t.tn * t.nog;
    size_t ring = 2 * (size_t)g->stage_floats;
    size_t red  = (size_t)std::max(t.ks - 1, t.kc > 1 ? 1 : 0) * t.tn * t.th * t.tw * g->nt;
    g->smem_bytes = 4 * ((size_t)g->patch + std::max(ring, red));
    g->chunks_per_rank = cdiv(cdiv(s.C, t.tc), t.kc);
    g->ctas = (long long)g->n_ocb * g->tiles_x * g->tiles_y * g->img_groups * t.kc;
    if (g->ctas >= (1ll << 31)) { *why = "grid too large"; return TDC_ERR_TILE; }
    if (g->smem_bytes > (size_t)dev.smem_per_cta) { *why = "tile needs more shared memory than a CTA may have"; return TDC_ERR_SMEM; }
    return TDC_OK;
}

// Registers per thread the compiler gives each accumulator count (from ptxas -v of the
// instances; the occupancy estimate only needs the three classes).
static int regs_estimate(const Variant& v) {
    int nacc = v.tn * v.th * v.tw;
    return nacc > 64 ? (v.tn == 4 ? 224 : 255) : (nacc > 32 ? 128 : 104);
}

static int ctas_per_sm(const Variant& v, const Geometry& g, const tdc_devinfo& dev) {
    int warps = cdiv(g.threads, 32);
    int by_regs = dev.regs_per_sm / (rup(regs_estimate(v), 8) * warps * 32);
    int by_smem = (int)((size_t)(dev.smem_per_cta + 1024) / (g.smem_bytes + 1024));
    int by_thr  = dev.threads_per_sm / (warps * 32);
    return std::max(0, std::min(std::min(by_regs, by_smem), std::min(by_thr, 32)));
}

// Fraction of its issue slots a scheduler fills with `w` resident warps of this kernel.
// Shape from the scheduler's latency hiding, level fitted to a measured B200 sweep of
// 2,300 tiles (measured time / modelled time had median 1.55 before the fit).
static double issue_eff(double w) {
    double e;
    if (w <= 1.0) e = 0.60;
    else if (w <= 2.0) e = 0.60 + 0.20 * (w - 1.0);
    else if (w <= 3.0) e = 0.80 + 0.08 * (w - 2.0);
    else if (w <= 4.0) e = 0.88 + 0.04 * (w - 3.0);
    else e = 0.92;
    return e / 1.55;
}

double tile_cost(const Shape& s, const tdc_tile& t, const Geometry& g, const tdc_devinfo& dev, double* vols) {
    const Variant& v = *g.v;
    const int RS = s.R * s.S, ocb = t.tn * t.nog, nacc = t.tn * t.th * t.tw;
    const int nchunks = std::min(cdiv(s.C, t.tc), g.chunks_per_rank);   // chunks the busiest CTA of a cluster walks
    // instructions one thread issues per input channel it owns
    double fma = (double)nacc * RS;
    double w_lds = RS * t.tn / 4.0, in_lds;
    if (v.kh == 0) in_lds = (double)RS * t.tw;
    else {
        int rowlen = (t.tw - 1) * s.stride + s.S;
        bool vec = (t.tw * s.stride) % 4 == 0;
        int row_lds = vec ? rowlen / 4 + ((rowlen % 4) ? ((rowlen % 4 == 3) ? 2 : 1) : 0) : rowlen;
        in_lds = (double)((t.th - 1) * s.stride + s.R) * row_lds;
    }
    double per_ch = fma + w_lds + in_lds + (v.kh == 0 ? 6.0 * RS : 6.0);
    // shared-memory wavefronts one warp draws per channel: a 16-byte load returns 512 bytes
    // to the register file = 4 wavefronts of the 128 B/clk path, 8-byte 2, 4-byte 1
    double wave_ch = RS * t.tn;   // = RS * (tn/4) loads * 4
    if (v.kh == 0) wave_ch += (double)RS * t.tw;
    else {
        int rowlen = (t.tw - 1) * s.stride + s.S;
        bool vec = (t.tw * s.stride) % 4 == 0;
        int in_rows_thread = (t.th - 1) * s.stride + s.R;
        wave_ch += (double)in_rows_thread * (vec ? (rowlen / 4) * 4 + (rowlen % 4) : rowlen);
    }
    // channels a slice walks: chunks are split evenly, the ragged last chunk too
    double ch_per_thread = 0;
    for (int kc = 0; kc < nchunks; ++kc) ch_per_thread += cdiv(std::min(t.tc, s.C - kc * t.tc), t.ks);
    double loader = nchunks * ((double)t.tc * g.patch / g.threads * 7.0 +
                               (double)t.tc * RS * ocb / 4.0 / g.threads * 8.0 + 60.0);
    double reduce = (t.ks > 1 ? 2.5 * nacc * (t.ks - 1) : 0.0) + (t.kc > 1 ? 2500.0 + 8.0 * nacc * (t.kc - 1) : 0.0);
    double fixed = (double)g.patch / g.threads * 30.0 + 900.0 + 3.0 * nacc;
    double per_thread = ch_per_thread * per_ch + loader + reduce + fixed;

    int cps = ctas_per_sm(v, g, dev);
    if (cps <= 0) return 1e30;
    const int warps = cdiv(g.threads, 32);
    const double lsu_per_warp = ch_per_thread * wave_ch + nchunks * ((double)t.tc * g.patch / g.threads + (double)t.tc * RS * ocb / g.threads);
    auto batch_time = [&](int resident) {   // cycles for `resident` co-resident CTAs on one SM
        double wps = resident * warps / 4.0;
        double issue = per_thread * std::max(wps, 1.0) / issue_eff(wps);
        double lsu = lsu_per_warp * resident * warps / 0.6;
        return std::max(issue, lsu) + 0.25 * std::min(issue, lsu);
    };
    // Latency of one CTA, which bounds a wave from below however few warps share the SM.  Each chunk is a dependent
    // step — copy issued, copy landed, barrier, arithmetic — and on a GPU that the grid barely fills (the batch-1
    // layers) nothing else hides it: 6,000 cycles a chunk plus its bytes at 20 B/clk, 0.7 of the chunk's arithmetic
    // on top (the rest runs under the next copy), and 70 cycles per accumulator for every further rank of a cluster
    // whose partial sums the leader adds over distributed shared memory.  Without this term the model kept few CTAs
    // walking many chunks where a cluster that splits them is 2x faster.  Constants chosen on a B200 by timing the
    // model's own pick for the 78 shapes of the measured tables (batch 1 to 256): it is 1.19x slower than the
    // table's tile on average (geometric mean over the six tables), against 1.37x without the term.
    const double chunk_bytes = 4.0 * ((double)t.tc * g.patch + (double)t.tc * RS * ocb);
    const double chunk_copy = 6000.0 + chunk_bytes / 20.0;
    const double chunk_math = (ch_per_thread / std::max(nchunks, 1)) * per_ch * std::max(warps / 4.0, 1.0) / issue_eff(warps / 4.0);
    const double cta_latency = nchunks * (chunk_copy + 0.7 * chunk_math) + fixed + (t.ks > 1 ? 2.5 * nacc * (t.ks - 1) : 0.0) +
                               (t.kc > 1 ? 70.0 * nacc * (t.kc - 1) : 0.0);
    long long slots = (long long)dev.sm_count * cps;
    long long full = g.ctas / slots, rem = g.ctas % slots;
    double cycles = full * std::max(batch_time(cps), cta_latency);
    if (rem) cycles += std::max(batch_time((int)cdiv((int)rem, dev.sm_count)), cta_latency);
    if (vols) {
        vols[0] = (double)g.ctas * s.C * RS * ocb;                 // filter words staged
        vols[1] = (double)g.ctas * s.C * g.patch;                  // input words staged
        vols[2] = (double)s.B * s.K * s.Ho() * s.Wo();             // output words written
        vols[3] = ch_per_thread * fma * (double)(full + (rem ? 1 : 0));   // flops * waves
    }
    return cycles;
}

static void push_unique(std::vector<int>* v, int x) {
    if (x > 0 && std::find(v->begin(), v->end(), x) == v->end()) v->push_back(x);
}

int select_tile(const Shape& s, const tdc_devinfo& dev, const tdc_tile& fx, tdc_tile* out) {
    const int Ho = s.Ho(), Wo = s.Wo();
    double best = 1e300;
    tdc_tile bt{};
    bool have_exact = false;
    for (const Variant* v : registry()) have_exact |= variant_fits(*v, s, true);
    for (const Variant* v : registry()) {
        if (!variant_fits(*v, s, have_exact)) continue;
        if ((fx.th && fx.th != v->th) || (fx.tw && fx.tw != v->tw) || (fx.tn && fx.tn != v->tn) ||
            (fx.nog && fx.nog != v->nog)) continue;
        if (v->tn * v->nog > rup(s.K, v->tn) && v->nog > 4) continue;   // CTA wider than the layer
        const int GY = cdiv(Ho, v->th), GX = cdiv(Wo, v->tw);
        std::vector<int> gys, gxs;
        if (fx.gy) gys.push_back(fx.gy); else for (int n = 1; n <= GY; ++n) push_unique(&gys, cdiv(GY, n));
        if (fx.gx) gxs.push_back(fx.gx); else for (int n = 1; n <= GX; ++n) push_unique(&gxs, cdiv(GX, n));
        for (int gy : gys) for (int gx : gxs) {
            std::vector<int> ims;
            if (fx.imgs) ims.push_back(fx.imgs);
            else {
                ims.push_back(1);
                if (gy * v->th >= Ho && gx * v->tw >= Wo)
                    for (int m : {2, 3, 4, 5, 6, 7, 8, 10, 12, 14, 16}) if (m <= s.B) ims.push_back(m);
            }
            for (int im : ims) {
                const int nt = v->nog * im * gy * gx;
                if (nt > v->maxt) continue;
                std::vector<int> kss;
                if (fx.ks) kss.push_back(fx.ks); else for (int k : {1, 2, 4, 8}) if (k <= s.C) kss.push_back(k);
                for (int ks : kss) {
                    const int thr = nt * ks;
                    if (thr > v->maxt) continue;
                    const long long base_ctas = (long long)cdiv(s.K, v->tn * v->nog) * cdiv(Ho, gy * v->th) *
                                                cdiv(Wo, gx * v->tw) * cdiv(s.B, im);
                    std::vector<int> kcs;
                    if (fx.kc) kcs.push_back(fx.kc);
                    else { kcs.push_back(1); if (base_ctas < 2 * dev.sm_count) for (int k : {2, 4, 8}) kcs.push_back(k); }
                    for (int kcl : kcs) {
                    std::vector<int> tcs;
                    if (fx.tc) tcs.push_back(fx.tc);
                    else for (int c : {4, 8, 16, 32}) if (c % ks == 0 && (c <= s.C || c == rup(std::min(c, s.C), ks))) tcs.push_back(c);
                    if (tcs.empty()) tcs.push_back(rup(std::min(4, s.C), ks));
                    for (int tc : tcs) {
                        if (kcl > 1 && cdiv(s.C, tc) < kcl) continue;   // fewer chunks than ranks
                        tdc_tile t{v->th, v->tw, tc, v->tn, v->nog, gy, gx, im, ks, kcl};
                        Geometry g;
                        if (make_geometry(s, t, dev, &g, nullptr) != TDC_OK) continue;
                        double c = tile_cost(s, t, g, dev, nullptr);
                        if (c < best) { best = c; bt = t; }
                    }
                    }
                }
            }
        }
    }
    if (best >= 1e299) return TDC_ERR_TILE;
    *out = bt;
    return TDC_OK;
}

}  // namespace tdc
