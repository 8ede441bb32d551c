// Prints the byte offset of every (row, 16-element block) scale factor as CUTLASS lays them out for the
// sm_100 block-scaled GEMM (cutlass::detail::Sm1xxBlockScaledConfig<16>, the layout the reference obtains at
// csrc/quantize/quantize_fp4_sfa.cu:191-206 and csrc/quantize/reshape_scales_sfa.cu:40-56).
// Host-only program: built and run by make_sf_layout_golden.py to produce sf_layout.npz.
// usage: sf_layout_table <rows> <K> <is_sfb>   -> first line = buffer size, then rows * K/16 offsets
#include <cstdio>
#include "cutlass/cutlass.h"
#include "cute/tensor.hpp"
#include "cutlass/detail/sm100_blockscaled_layout.hpp"
using Cfg = cutlass::detail::Sm1xxBlockScaledConfig<16>;
int main(int argc, char** argv) {
    int rows = atoi(argv[1]), K = atoi(argv[2]), is_b = atoi(argv[3]);
    auto shape = is_b ? cute::make_shape(1, rows, K, 1) : cute::make_shape(rows, 1, K, 1);
    if (is_b) {
        auto layout = Cfg::tile_atom_to_shape_SFB(shape);
        printf("%d\n", (int)cute::cosize(layout));
        for (int r = 0; r < rows; ++r) for (int b = 0; b < K / 16; ++b) printf("%d\n", (int)layout(r, b * 16, 0));
    } else {
        auto layout = Cfg::tile_atom_to_shape_SFA(shape);
        printf("%d\n", (int)cute::cosize(layout));
        for (int r = 0; r < rows; ++r) for (int b = 0; b < K / 16; ++b) printf("%d\n", (int)layout(r, b * 16, 0));
    }
    return 0;
}
