// Host interface of the tcgen05 implicit-GEMM convolution (conv_tc.cu).
#pragma once

#include <cuda.h>

#include "conv_common.cuh"

namespace tsb {
namespace tc {

struct Config {
    int bn = 0, bk = 0;               // tile width in output channels, K block in bytes (= swizzle span)
    int num_m_tiles = 0, num_n_tiles = 0;
    int grid = 0;                     // persistent CTAs
};

// Whether the tensor-core kernel covers this geometry; *why names the reason when it does not.
bool supported(const ConvGeom &g, const char **why);
Config choose_config(const ConvGeom &g, int sm_count);
// w_packed: [O][KH][KW][Cp] int8
int encode_weight_map(const ConvGeom &g, const Config &cfg, const int8_t *w_packed, CUtensorMap *map);
// x_nhwc: [N][H][W][Cp] int8, 16-byte aligned
int encode_activation_map(const ConvGeom &g, const Config &cfg, const int8_t *x_nhwc, CUtensorMap *map);
int launch_conv_tc(const ConvGeom &g, const Config &cfg, const CUtensorMap &map_a, const CUtensorMap &map_b,
                   const EpiParams &epi, int *status_word, cudaStream_t stream);

}  // namespace tc
}  // namespace tsb
