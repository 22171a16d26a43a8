// Host-side helpers shared by the translation units of libfp4b200: error reporting for the
// C ABI, CUDA error checking, device properties, tensor-map encoding, the device status word.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

namespace fp4b200 {

// Records a printf-style message retrievable through fp4b200_last_error(); returns -1.
int set_error(const char* fmt, ...);

#define FP4_CUDA_CHECK(expr)                                                                    \
  do {                                                                                          \
    cudaError_t _e = (expr);                                                                    \
    if (_e != cudaSuccess)                                                                      \
      return ::fp4b200::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
  } while (0)

int device_sm_count();

// Device address of the per-device status word array (4 ints); nullptr + error on failure.
int* device_status_ptr();

// Device scratch of kScratchFloats floats private to (current device, stream).  Kernels of one stream
// run in order, so consecutive launches of one entry point may hand small results to each other
// through it (per-CTA partial maxima of a pass-1 kernel, read by the kernel launched next).  Allocated
// with cudaMalloc on the first use of a stream and kept for the life of the process; nullptr + error
// on failure (e.g. a first use inside a stream capture).
constexpr int kScratchFloats = 2048;
float* stream_scratch(cudaStream_t st);

// Per-CTA partial tensor maxima left in scratch by a pass-1 kernel for the kernel launched next.
struct AmaxPartials {
  const float* ptr = nullptr;
  int count = 0;
};

// Encodes a 2-D tiled tensor map: inner extent dim0 (elements), outer extent dim1, row pitch
// in bytes, box (box0 x box1) elements.  Returns 0 or -1 (message set).
int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t dim0,
                 uint64_t dim1, uint64_t pitch_bytes, uint32_t box0, uint32_t box1, CUtensorMapSwizzle swizzle);

// Options of the stochastic-rounding / Hadamard variants of the NVFP4 quantiser (one launch).
struct QuantOpt {
  int sr_row, sr_col;        // data stochastic rounding of the row pass / of the column pass
  int scale_sr;              // stochastic rounding of the E4M3 scale byte (one more random word per block, drawn first)
  int row_per_stage;         // 0: by the launch's shape; 8: the row pass follows a row-only launch's random stream
  int rht_row, rht_col;      // 16-point Hadamard transform along K (row operand) / along M (column operand)
  int sign;                  // seeded sign flip before the transform
  int return_row;            // 0: skip the row-wise outputs but keep their place in the random stream
  unsigned long long rng_seed, rng_offset, rng_offset_col;   // column pass may take its own counter offset
  const void* rng_state;     // device words {key, base} (8-byte aligned) or null: the key replaces rng_seed, base is added to both offsets
  unsigned long long sign_seed, sign_subseq;
  // encode-centric scale_sr: 2 * (M/128) * (K/128) * 128 uint16 of device scratch for the map of blocks that draw no
  // scale word (null: every block is taken to draw one)
  void* ec_zero_scratch;
};

// Launchers defined in quant_nvfp4.cu and shared with the other producers.
// Tensor amax of a bf16 buffer.  partials_out == nullptr: amax_sg[0] = max|x|, amax_sg[1] = amax/2688
// are written on the stream (two launches).  Otherwise only the per-CTA maxima are produced, in
// `scratch` (kScratchFloats floats), described by *partials_out, for a quantiser launched next.
int launch_amax(const void* x, int64_t n_elems, float* amax_sg, cudaStream_t st, float* scratch = nullptr,
                AmaxPartials* partials_out = nullptr);
// Row (+ column when col_* non-null) NVFP4 quantisation; RMSNorm is applied on the fly when
// inv_rms/gamma are given; reverse walks the chunks back to front; weight_2d shares one scale per
// 16x16 tile between the two orientations (decode-centric).
// The tensor amax comes either from the device scalars amax_row / amax_col, or (partials != nullptr)
// from the partial maxima of this library's own pass-1 kernel launched just before on st over the
// same x, which it only reads: the quantiser is then launched programmatically dependent on that
// kernel (it fetches its first chunks while that kernel drains), reduces the partials itself and
// writes amax_out[0] = amax, amax_out[1] = amax/2688 (when non-null).  sg_out (when non-null)
// receives amax_row/2688 in both cases.  nhsd_seq > 0: x is laid out [B, nhsd_heads, nhsd_seq, 64] and
// stands for the matrix [M = B * nhsd_seq, K = nhsd_heads * 64]; row_pitch_bytes > 0: row_fp4 is a column slice
// of a wider code matrix with that pitch (both: plain quantisation only).
int launch_quantize(const void* x, int64_t M, int64_t K, const float* amax_row, const float* amax_col,
                    bool encode_centric, const float* inv_rms, const void* gamma, void* row_fp4, void* row_sc,
                    void* col_fp4, void* col_sc, float* sg_out, bool reverse, cudaStream_t st, bool weight_2d = false,
                    const QuantOpt* opt = nullptr, const AmaxPartials* partials = nullptr, float* amax_out = nullptr,
                    int nhsd_heads = 0, int nhsd_seq = 0, int64_t row_pitch_bytes = 0);

}  // namespace fp4b200
