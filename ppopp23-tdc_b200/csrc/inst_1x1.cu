// Instances of conv_f32_kernel for one filter family; see variants.h.
#include "variants.h"

namespace tdc {
static const Variant k_table[] = {TDC_FOR_ALL_TILES(TDC_VARIANT, 1, 1, 1)};
const Variant* variants_1x1(int* n) {
    *n = (int)(sizeof(k_table) / sizeof(k_table[0]));
    return k_table;
}
}  // namespace tdc
