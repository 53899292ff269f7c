// Host interface of the tcgen05 implicit-GEMM convolution (conv_tc.cu).
#pragma once

#include <cuda.h>

#include "conv_common.cuh"

namespace tsb {
namespace tc {

// The convolution as the tensor-core kernel sees it.
//  fold == 0: activations are NHWC_PAD [N][H][W][Cp]; `g` is the real geometry.
//  fold == 1 (at most 16 input channels): activations are staged as [N][H][Wp][cpix] with pixel w at column
//            w + pad_left and zeros elsewhere.  The KW taps of one filter row are then one contiguous run of bytes,
//            so the kernel sees a KH x 1 filter over `g.Cp` = round_up(((KW-1)*dw+1)*cpix, 64) virtual channels whose
//            pixel stride is stride_w*cpix bytes (the tensor map's rows overlap); `g` is that virtual geometry.
//  rows == 1 (a fold view whose pixel stride is exactly 16 bytes and whose output rows are long): "raw-row" mode.  A tile
//            is up to 128 consecutive pixels of one output row; per filter row the kernel copies the staged bytes under
//            those pixels ONCE (about 2 KB instead of 128 windows of 64 B) and the MMA reads the overlapping windows
//            straight out of that copy through a no-swizzle descriptor whose rows are 16 bytes apart.
//  patch == 1 (NHWC_PAD input, stride 1, more than one filter tap): the configuration may use "patch" mode.  A tile is
//            8 pixels wide and pix/8 pixels high; one tiled tensor-map load per channel block brings the input patch under
//            it (halo included, zero-filled outside the image) and every filter tap reads its shifted window out of that
//            patch, so an activation byte is loaded once per tile instead of once per tap.  Needs resident weights.
struct View {
    ConvGeom g;          // geometry handed to the kernel and the tensor maps
    ConvGeom real;       // geometry of the operator
    int fold = 0;
    int rows = 0;        // raw-row mode
    int patch = 0;       // patch mode is possible for this geometry
    int rows_segs = 0;   // tiles per output row in raw-row mode
    int a_tiled = 0;     // 1x1 / stride 1 / no padding: the activations are the [M][Cp] matrix itself, loaded as 2-D tiles
    int cpix = 0;        // bytes per pixel of the folded staging
    int Wp = 0;          // pixels per row of the folded staging
    uint64_t stride_w = 0, stride_h = 0, stride_n = 0;  // bytes between neighbours along W, H, N as the tensor map sees them
    size_t stage_bytes = 0;    // NHWC_PAD or folded staging of one input
    size_t weight_bytes = 0;   // packed weights
};

struct Config {
    int bn = 0, bk = 0;               // N of the MMA instruction, K block in bytes (= swizzle span)
    int swap = 0;                     // 1: channels on the MMA's M side and pixels on its N side
    int pix = 0, ch = 0;              // pixels and output channels per tile
    int num_m_tiles = 0, num_n_tiles = 0;
    int patch = 0;                    // this configuration runs in patch mode
    int patch_tiles_w = 0, patch_tiles_h = 0, patch_pw = 0, patch_ph = 0;   // tiles per image, patch extent in pixels
    int grid = 0;                     // persistent CTAs
    // shared-memory plan of the kernel
    int stages = 0, b_resident = 0;
    int kgroup = 1;                   // K blocks per pipeline stage (im2col / tiled loads; 1 in patch and raw-row mode)
    uint32_t unit_bytes = 0;          // one K block of a stage
    uint32_t stage_bytes = 0, b_off = 0, bar_off = 0, dyn_smem = 0;
    int staging = 0;                  // shared memory set aside for the staged epilogue: 0 none, 1 int8 tiles, 2 fp32 + int8 tiles
    uint32_t stg_off = 0;
};

// Overrides of the plan heuristics, from tsb_conv_desc (tests force every code path with them): 0 = the library
// chooses, 1 = off / normal orientation, 2 = on / swapped orientation.
struct Tuning {
    int orientation = 0;   // TSB_TUNE_* of tsb_conv_desc::mma_orientation
    int rows = 0;          // tsb_conv_desc::raw_row_mode
    int patch = 0;         // tsb_conv_desc::patch_mode
};

// Whether the tensor-core kernel covers this geometry; *why names the reason when it does not.
bool make_view(const ConvGeom &g, const Tuning &tune, View *view, const char **why);
// orientation: -1 = by heuristic (or tune.orientation), 0 = normal, 1 = swapped (any number of output channels, 128
// per channel tile)
// staging: shared memory to set aside for the staged epilogue (see Config::staging); only normal-orientation
// configurations use it
Config choose_config(const View &v, const Tuning &tune, int sm_count, int orientation, int staging = 0);
// Which staged epilogue these outputs can take with this view: 0 none (direct stores), 1 int8 NHWC_PAD tile only,
// 2 pixel-major fp32 residual / output (and int8) tiles.
int staging_level(const View &v, const EpiParams &epi);
// w_packed: [O][KH][KW][Cp] int8 of the view's geometry
int encode_weight_map(const View &v, const Config &cfg, const int8_t *w_packed, CUtensorMap *map);
// x: the staged activations (NHWC_PAD or folded), 16-byte aligned
int encode_activation_map(const View &v, const Config &cfg, const int8_t *x, CUtensorMap *map);
// OIHW weights -> the packed layout of the view
int pack_weights(const View &v, const int8_t *w_oihw, int8_t *w_packed, cudaStream_t stream);
// int8 input (NCHW, or NHWC_PAD when x_nhwc) -> folded staging (fold views only)
int stage_folded(const View &v, const int8_t *x, int x_nhwc, int8_t *staged, cudaStream_t stream);
#ifdef TSB_ENABLE_TRACE
// Profiling builds only: CTA 0 of later launches writes 8 time stamps (ns) per tile for its first 32 tiles into this
// device buffer of 256 x 8 bytes; null switches it off.
void set_trace_buffer(unsigned long long *device_buffer);
#endif
// A projection shortcut run inside the main convolution's kernel: a 1x1 convolution (any stride, no padding) over the
// same output pixels, whose dequantized (+ bias) result is the main convolution's residual.  Both tensor maps are
// encoded with the configuration of choose_config_dual.
struct DualArgs {
    const View *view;          // the projection
    CUtensorMap map_a, map_b;  // its staged activations and packed weights
    const float *dq, *bias;    // its dequantize scales and bias (may be null), per output channel, device pointers
                               // dq == null: channel concatenation -- `view` convolves the FIRST part of the concatenated input
                               // and its K blocks are summed into the main convolution's accumulator; no residual
};
// whether `shortcut` can run inside the kernel of `v`; *why names the reason when it cannot
bool dual_supported(const View &v, const View &shortcut, const char **why);
// one configuration for the pair: common K block, both weight tiles resident when they fit; bn: 0 = by output channels
Config choose_config_dual(const View &v, const View &shortcut, int sm_count, int bn, bool concat = false);
// x_staged: the activations the map_a was encoded for (read directly in raw-row mode)
int launch_conv_tc(const View &v, const Config &cfg, const CUtensorMap &map_a, const CUtensorMap &map_b,
                   const int8_t *x_staged, const EpiParams &epi, int *status_word, cudaStream_t stream,
                   const DualArgs *dual = nullptr);

}  // namespace tc
}  // namespace tsb
