// A chain of quantised linear layers over at most 64 rows (an INT8 MLP at serving batch sizes) as ONE
// cooperative tcgen05 kernel: parameters shared by the host side (kernels_umma.cu) and the kernel (umma_chain.cu).
//
// With so few rows a layer is a stream of its weights: 2 * rows operations per weight byte.  The roles of the
// two MMA operands are therefore swapped against the convolution kernel: the WEIGHTS are the 128-row operand
// (128 output channels per tile) and the activation rows are the N = 64 columns, so a work unit is
// (128 channels) x (a slice of K), its accumulator 128 lanes x 64 columns of TMEM, and every CTA of the grid
// owns at most one unit per layer.  Every slice of K leaves its partial sums in an L2-resident workspace;
// the unit that arrives last at a channel tile adds them, requantises and writes the next layer's activation rows; one grid-wide barrier separates two layers.  Weights do not depend on activations, so every
// CTA starts the loads of all its weight slices that fit in shared memory at kernel entry: HBM streams
// through the barriers.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace oxb {
namespace k {
namespace umma {

constexpr int CHAIN_MAX_LAYERS = 4;
constexpr int CHAIN_ROWS = 64;                  // MMA N: activation rows per launch (fewer are zero-filled by TMA)
constexpr int CHAIN_W_TILE = 128 * 128;         // bytes of one K block of a weight slice: 128 channels x 128 bytes of K
constexpr int CHAIN_X_TILE = CHAIN_ROWS * 128;  // bytes of one K block of the activation rows
constexpr int CHAIN_THREADS = 160;              // warps 0..3: accumulator lanes 32w..32w+31; warp 4: TMA and MMA issue

struct alignas(64) ChainLayerParams {
  CUtensorMap tmW;  // the weights repacked [channel tile][K block][128 channels][128 bytes of K], seen as rows of 128 bytes; box 128 x 128, 128-byte swizzle
  CUtensorMap tmX;  // [rows][K] 8-bit activations, box 128 bytes of K x 64 rows, 128-byte swizzle
  int N;
  int n_tiles, splits;  // unit u < n_tiles * splits is (channel tile u / splits, K slice u % splits)
  int kb;               // K blocks (128 bytes of K each) per unit
  uint32_t idesc;
  uint32_t w_off;  // byte offset of this layer's weight region in the CTA's shared memory
  int w_after;     // -1: the region is this layer's from kernel entry; j: it is layer j's until j's MMAs have completed
  const int32_t* bias_i;  // [N] bias with the input zero point folded in: acc = sum(x * w) + bias_i
  const float* combined;  // [N] x_scale * w_scale[ch] / y_scale
  int y_zp, lo, hi;
  uint8_t* out;              // [rows][N] 8-bit lanes: the next layer's activation rows
  int fma_exact;             // the one-FMA requantisation is exact for every scale of this layer (accumulators below 2^24)
  int32_t* ws;               // [n_tiles][splits][16][128][4] partial sums of the K slices (rows / 4, channel, rows % 4)
  unsigned int* tile_count;  // [n_tiles] arrivals; zero between launches
};

struct alignas(64) ChainParams {
  ChainLayerParams layer[CHAIN_MAX_LAYERS];
  int n_layers, rows;
  int cluster;  // > 1: the K slices of a channel tile are the CTAs of one cluster of this size (splits == cluster in every layer)
  uint32_t x_off;          // byte offset of the activation region (reused by every layer)
  // optional ends: a QuantizeLinear in front of the first layer (f32 rows of head_k lanes) and a DequantizeLinear
  // behind the last one (f32 [rows][N] beside the 8-bit rows)
  const float* head_x;
  uint8_t* head_q;  // the first layer's 8-bit rows, [rows][head_k]
  int head_k;
  float head_scale, head_zp, head_lo, head_hi;
  float* tail_out;
  float tail_scale, tail_zp;
  int tail_signed;
  unsigned long long* grid_bar;  // arrivals at the grid-wide barrier since the scratch was cleared
  int* err_flag;
};

// false when the driver refuses the launch (nothing ran)
// repacks [N][K] 8-bit weights (K a multiple of 128) into the tile order tmW describes; out holds ceil(N / 128) * 128 * K bytes
void chain_repack(const void* w, void* out, int N, int K, cudaStream_t s);
bool launch_chain(const ChainParams& p, int grid, size_t smem, int device, int cluster, cudaStream_t s);
// One launch with no layers (the kernel sets up and leaves) on the default stream, waited for: false when the driver
// refuses the geometry (cooperative launch of clusters) or the launch fails.
bool try_launch_chain(const ChainParams& p, int grid, size_t smem, int device, int cluster);
// CTAs of the chain kernel that can be resident at once on `device` with `smem` bytes of dynamic shared memory
int chain_max_resident(size_t smem, int device, int cluster);

}  // namespace umma
}  // namespace k
}  // namespace oxb
