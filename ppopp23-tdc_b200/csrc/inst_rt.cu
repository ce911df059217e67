// Instances of conv_f32_kernel for one filter family; see variants.h.
#include "variants.h"

namespace tdc {
static const Variant k_table[] = {TDC_FOR_ROW_TILES(TDC_VARIANT, 0, 0, 1), TDC_FOR_ROW_TILES(TDC_VARIANT, 0, 0, 2)};
const Variant* variants_rt(int* n) {
    *n = (int)(sizeof(k_table) / sizeof(k_table[0]));
    return k_table;
}
}  // namespace tdc
