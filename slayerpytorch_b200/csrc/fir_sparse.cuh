// Event-driven temporal filter for mostly-zero inputs (fir_sparse.cu), as fir.cu calls it.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace sb200 {

constexpr int64_t kFirSparseMaxT = 4096;        // 8 bytes of event list per sample and warp
constexpr int64_t kFirSparseMaxTaps = 1024;
// The event-driven kernel is chosen when at most this many of 1024 sampled input samples are
// non-zero: the measured cross-over against the dense scalar kernel, for 77 taps - 6 % on fp32
// input, 9 % on packed input (whose event list comes cheaper).
constexpr int kFirSparseMaxPer1024 = 61;
constexpr int kFirSparseMaxPer1024Bits = 92;

// Shapes the event-driven kernel takes.
bool fir_sparse_eligible(int64_t rows, int64_t T, int64_t K);

// Enqueues the density probe over an input of `rows` rows of T samples (fp32, or packed spikes
// when `bits`); *flag then points to a device word that is 1 if the event-driven kernel should run
// and 0 if the dense one should, or is NULL when no scratch could be had (run the dense kernel).
int fir_sparse_probe(const void *in, int64_t rows, int64_t T, bool bits, const float *filt, int64_t K,
                     cudaStream_t stream, const int **flag);

// Enqueues the event-driven kernel; with run_flag != NULL it returns at once unless *run_flag != 0.
int fir_sparse_launch(int dir, bool bits, float *out, const void *in, const float *filt, int64_t rows, int64_t T,
                      int64_t K, float Ts, float spike_value, const int *run_flag, cudaStream_t stream);

}  // namespace sb200
