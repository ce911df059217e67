// Host-side geometry of a (shape, tile) pair and the analytical tile selector.
// Pure C++ (no CUDA calls) so it can be exercised without a GPU.
#pragma once
#include <stddef.h>
#include "../../include/tdc_b200.h"
#include "variants.h"

namespace tdc {

struct Shape {
    int B, C, H, W, K, R, S, pad, stride;
    int Ho() const { return (H + 2 * pad - R) / stride + 1; }
    int Wo() const { return (W + 2 * pad - S) / stride + 1; }
};

// Everything the launch needs that follows from shape + completed tile.
struct Geometry {
    const Variant* v;
    int in_rows, in_w, in_wp, patch;
    int tiles_y, tiles_x, img_groups, n_ocb;
    int threads, nt;           // threads per CTA, threads of one channel slice
    int stage_floats;
    int chunks_per_rank;       // channel chunks each CTA of a cluster walks
    size_t smem_bytes;
    long long ctas;
};

const Variant* find_variant(const Shape& s, const tdc_tile& t);

// Fills `g` for a tile whose fields are all non-zero. Returns TDC_OK or the reason the
// pair is invalid (message in *why when given).
int make_geometry(const Shape& s, const tdc_tile& t, const tdc_devinfo& dev, Geometry* g,
                  const char** why);

// Modelled run time in SM cycles; vols = {filter volume, input volume, output volume,
// flops*waves} in the sense of TDC-LAYERS-MODELING/model.py:135-184.
double tile_cost(const Shape& s, const tdc_tile& t, const Geometry& g, const tdc_devinfo& dev,
                 double* vols);

// Best tile under the model among all compiled variants; fields of `fixed` that are
// non-zero are kept as given. Returns TDC_OK or TDC_ERR_TILE when nothing fits.
int select_tile(const Shape& s, const tdc_devinfo& dev, const tdc_tile& fixed, tdc_tile* out);

}  // namespace tdc
