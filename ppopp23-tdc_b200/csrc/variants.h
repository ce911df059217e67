// Registry of the compiled instances of conv_f32_kernel.  The reference emits one
// source file per (shape, TH, TW, TC) by text substitution
// (A100-evaluation/TDC-LAYERS-ORACLE/gen_from_occupancy.py:113-139); here a fixed set of
// thread tiles is compiled once and the shape, TC and the CTA geometry are run-time
// arguments.
#pragma once
#include "core_conv_f32.cuh"

namespace tdc {

struct Variant {
    int kh, kw, stride;   // kh == 0: filter size is a run-time argument (th must be 1)
    int tn, th, tw, nog;
    int maxt;             // __launch_bounds__ of the instance
    const void* fn;
};

// Each instantiation file returns its own slice of the registry.
const Variant* variants_3x3s1(int* n);
const Variant* variants_3x3s2(int* n);
const Variant* variants_1x1(int* n);
const Variant* variants_rt(int* n);

// Threads a thread tile may be launched with: tiles with more than 64 accumulators
// need the whole register budget of a 256-thread CTA.
constexpr int maxt_for(int tn, int th, int tw) { return (tn * th * tw > 64) ? 256 : 512; }

#define TDC_VARIANT(KH, KW, ST, TN, TH, TW, NOG)                                                  \
    Variant {                                                                                     \
        KH, KW, ST, TN, TH, TW, NOG, maxt_for(TN, TH, TW),                                        \
            (const void*)&conv_f32_kernel<KH, KW, ST, TN, TH, TW, NOG, maxt_for(TN, TH, TW)>      \
    }

// The thread tiles every filter family is compiled for: (TN, TH, TW, NOG).
#define TDC_FOR_ALL_TILES(X, KH, KW, ST)                                                          \
    X(KH, KW, ST, 4, 4, 8, 8), X(KH, KW, ST, 4, 4, 8, 16), X(KH, KW, ST, 4, 4, 7, 8),             \
    X(KH, KW, ST, 4, 4, 7, 16), X(KH, KW, ST, 8, 2, 8, 4), X(KH, KW, ST, 8, 2, 8, 8),             \
    X(KH, KW, ST, 8, 2, 7, 4), X(KH, KW, ST, 8, 2, 7, 8), X(KH, KW, ST, 4, 2, 8, 8),              \
    X(KH, KW, ST, 4, 2, 8, 16), X(KH, KW, ST, 4, 2, 7, 8), X(KH, KW, ST, 4, 2, 7, 16),            \
    X(KH, KW, ST, 8, 1, 8, 4), X(KH, KW, ST, 8, 1, 8, 8), X(KH, KW, ST, 8, 1, 7, 4),              \
    X(KH, KW, ST, 8, 1, 7, 8), X(KH, KW, ST, 4, 1, 8, 4), X(KH, KW, ST, 4, 1, 8, 8),              \
    X(KH, KW, ST, 4, 1, 7, 4), X(KH, KW, ST, 4, 1, 7, 8)

#define TDC_FOR_ROW_TILES(X, KH, KW, ST)                                                          \
    X(KH, KW, ST, 8, 1, 7, 4), X(KH, KW, ST, 8, 1, 7, 8), X(KH, KW, ST, 8, 1, 8, 4),              \
    X(KH, KW, ST, 8, 1, 8, 8), X(KH, KW, ST, 4, 1, 7, 4), X(KH, KW, ST, 4, 1, 7, 8),              \
    X(KH, KW, ST, 4, 1, 8, 4), X(KH, KW, ST, 4, 1, 8, 8)

}  // namespace tdc
