/*
 * slayer_b200 — C ABI of the Blackwell (sm_100a) SLAYER spiking-neuron operators.
 *
 * Every entry point takes plain device pointers and sizes; no framework types cross this
 * boundary.  All tensors are float32, row-major [rows, T] with time last and contiguous,
 * resident on the CUDA device that is current on the calling thread.  `stream` is a
 * cudaStream_t passed as void* (NULL = the legacy default stream).  Calls are asynchronous
 * with respect to the host: they enqueue work on `stream` and return.
 *
 * Return value: 0 on success, a negative SLAYER_B200_E* code on failure.  After a failure,
 * slayer_b200_last_error() returns a human-readable message for the calling thread.
 * Nothing here falls back to the CPU: without a usable GPU the calls fail.
 *
 * The Python extension modules `slayerCuda` and `slayerLoihiCuda` built from this library
 * export the reference's operator names and signatures on top of these functions.
 */
#ifndef SLAYER_B200_H_INCLUDED
#define SLAYER_B200_H_INCLUDED

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SLAYER_B200_OK          0
#define SLAYER_B200_EINVAL     -1   /* bad argument (null pointer, negative size, ...)      */
#define SLAYER_B200_ECUDA      -2   /* a CUDA runtime call or kernel launch failed          */
#define SLAYER_B200_EUNSUPPORTED -3 /* argument outside what the kernels implement          */
#define SLAYER_B200_EDEVICE    -4   /* a kernel reported a device-side error status         */

/* ABI version of this header (bumped when a signature changes). */
int slayer_b200_abi_version(void);

/* Message describing the last failure on the calling thread ("" if none). */
const char *slayer_b200_last_error(void);

/*
 * Causal temporal FIR (psp filter):  out[r,t] = Ts * sum_{i<K, i<=t} in[r,t-i] * filter[i].
 * fp32 fused multiply-add chain in ascending tap order, one multiply by Ts at the end.
 * Replaces conv<float>() / convKernel, src/cuda/convKernels.h:10-35, :64-96, reached from
 * convCuda, src/cuda/slayerKernels.cu:41-57.  `out` must not alias `in`.
 */
int slayer_b200_conv(float *out, const float *in, const float *filter,
                     int64_t rows, int64_t T, int64_t K, float Ts, void *stream);

/*
 * Adjoint of the above:  out[r,t] = Ts * sum_{i<K, t+i<T} in[r,t+i] * filter[i].
 * Replaces corr<float>() / corrKernel, src/cuda/convKernels.h:37-62, :98-129, reached from
 * corrCuda, src/cuda/slayerKernels.cu:59-75.  `out` must not alias `in`.
 */
int slayer_b200_corr(float *out, const float *in, const float *filter,
                     int64_t rows, int64_t T, int64_t K, float Ts, void *stream);

/*
 * slayer_b200_corr followed by slayer_b200_spike_grad on its result, in one pass:
 *   out[r,t] = (Ts * sum_{i<K, t+i<T} in[r,t+i] * filter[i]) * scale/tau * exp(-|u[r,t] - theta| / tau),
 * the backward step of "spike, then psp": pspFunction.backward / _pspFunction.backward (corr,
 * src/slayer.py:892) and then spikeFunction.backward (the tensor expression at src/slayer.py:862)
 * of the layer that produced the spikes, without the intermediate gradient tensor (12 instead of
 * 20 bytes per element).  The filtered value is rounded to fp32 before it is multiplied, so the
 * result equals the two calls', except that an exponential below 1.2e-38 is flushed to zero
 * (the filter's translation unit flushes denormals, the separate pass does not): a difference of
 * at most 1.2e-38 * scale/tau * |filtered value|.  `out` must alias neither `in` nor `u`.  It has no counterpart in the reference.
 */
int slayer_b200_corr_spike_grad(float *out, const float *in, const float *filter, const float *u,
                                int64_t rows, int64_t T, int64_t K, float Ts,
                                float theta, float tau, float scale, void *stream);

/*
 * Time shift by one amount for all rows:  out[r,t] = in[r,t-d] if 0 <= t-d < T else 0,
 * d = trunc(shift / Ts) (toward zero; negative shifts advance the signal).
 * Replaces shift<float>() scalar form / shiftKernel, src/cuda/shiftKernels.h:9-34, :63-98,
 * reached from shiftCuda (1-element branch) and shiftFlCuda, slayerKernels.cu:87-95, :115-129.
 */
int slayer_b200_shift_scalar(float *out, const float *in, float shift,
                             int64_t rows, int64_t T, float Ts, void *stream);

/*
 * Per-neuron time shift: rows = nBatch * nNeurons, row r uses lut[r % nNeurons] (device
 * pointer to nNeurons floats).  One launch covers the whole batch.
 * Replaces shift<float>() LUT form / shiftKernel, src/cuda/shiftKernels.h:36-61, :100-136,
 * reached from shiftCuda, src/cuda/slayerKernels.cu:96-105.
 */
int slayer_b200_shift_lut(float *out, const float *in, const float *lut,
                          int64_t nBatch, int64_t nNeurons, int64_t T, float Ts, void *stream);

/*
 * SRM spike generation with refractory response.  For each row, in time order:
 * if u[t] >= theta then s[t] = 1/Ts and nu[0..nuSize) is added into u[t..t+nuSize) (clipped
 * at T, one fp32 add per sample, in spike order); else s[t] = 0.  `u` is updated in place.
 * Spike positions and the updated u are bit-identical to the sequential definition.
 * Replaces getSpikes<float>() / getSpikesKernel, src/cuda/spikeKernels.h:9-38, :54-60,
 * reached from getSpikesCuda, src/cuda/slayerKernels.cu:14-39.
 */
int slayer_b200_srm_get_spikes(float *s, float *u, const float *nu,
                               int64_t rows, int64_t nuSize, int64_t T,
                               float theta, float Ts, void *stream);

/*
 * Loihi CUBA neuron (fixed-point current and voltage decay, threshold, refractory delay).
 * Input w[r,t] holds integer-valued weighted spikes; outputs are the spike train s (0/1),
 * the voltage v and the current u as float32 images of the int32 state.  Integer
 * arithmetic follows the reference's C++ promotion rules exactly (uint32 products with
 * wrap-around, logical >> 12).  refDelay must be >= 1.
 * Replaces getSpikes<float>() / getSpikesKernel, src/cuda/spikeLoihiKernels.h:9-72, :75-96,
 * reached from getSpikesCuda, src/cuda/slayerLoihiKernels.cu:12-46.
 */
int slayer_b200_loihi_get_spikes(float *s, float *v, float *u, const float *w,
                                 int64_t rows, int64_t T,
                                 uint32_t wgtExp, uint32_t theta, uint32_t iDecay,
                                 uint32_t vDecay, uint32_t refDelay, void *stream);

/*
 * slayer_b200_loihi_get_spikes followed by a delay of `delay` time steps (0 .. 63) on the spikes,
 * with the spikes written once, already delayed: delayed[r, t] = s[r, t - delay] (0 for
 * t < delay); v as above; u may be NULL, in which case the current is not written (callers that
 * keep only spikes and voltage, as _spike.forward does, src/slayerLoihi.py:257-262).  The same
 * bits as getSpikes<float>() (src/cuda/spikeLoihiKernels.h:75-96) followed by the scalar
 * shift<float>() (src/cuda/shiftKernels.h:63-98) that every Loihi layer applies with a delay of
 * one step (delayShift(spike, 1), exampleLoihi/03_IBMGesture/ibmGestureTrain.py:56-79); 12 instead
 * of 24 bytes per element.  Needs 16-byte aligned buffers and theta < 2^31, else
 * SLAYER_B200_EUNSUPPORTED (run the two calls instead).
 */
int slayer_b200_loihi_get_spikes_delayed(float *delayed, float *v, float *u, const float *w,
                                         int64_t rows, int64_t T,
                                         uint32_t wgtExp, uint32_t theta, uint32_t iDecay,
                                         uint32_t vDecay, uint32_t refDelay, int64_t delay, void *stream);

/*
 * Surrogate gradient of the spike function, fused into one pass:
 *   out[i] = g[i] * ( scale / tau * exp(-|u[i] - theta| / tau) ),   i < n.
 * `out` may alias `g`.  Replaces the chain of elementwise tensor operations in
 * _spikeFunction.backward, src/slayer.py:858-865, and _spike.backward,
 * src/slayerLoihi.py:279-283 (tau = tauRho * theta, scale = scaleRho); the reference's
 * never-bound native twin is evalRhoKernel, src/cuda/spikeKernels.h:41-52.
 */
int slayer_b200_spike_grad(float *out, const float *g, const float *u, int64_t n,
                           float theta, float tau, float scale, void *stream);

/*
 * Backward step of "spike, then delay" in one pass:
 *   out[b,n,t] = shifted(b,n,t) * scale/tau * exp(-|u[b,n,t] - theta| / tau),
 *   shifted(b,n,t) = grad_output[b,n,t - d_n] if 0 <= t - d_n < T else 0,
 *   d_n = trunc(shift_n / Ts),  shift_n = shift_lut[n] if shift_lut is not NULL, else `shift`.
 * The same result as slayer_b200_shift_lut / _scalar followed by slayer_b200_spike_grad, bit
 * for bit, without the intermediate tensor.  The caller passes the shift to apply to the
 * gradient, i.e. minus the forward delay (as _delayFunction.backward does, src/slayer.py:957,
 * before the expression at src/slayer.py:862).  out must not alias grad_output.
 */
int slayer_b200_spike_grad_shift(float *out, const float *grad_output, const float *u, const float *shift_lut,
                                 float shift, int64_t nBatch, int64_t nNeurons, int64_t T, float Ts,
                                 float theta, float tau, float scale, void *stream);

/*
 * Gradient with respect to per-neuron axonal delays, fused into one pass:
 *   grad_delay[n] = Ts * sum_{b,t} grad_output[b,n,t] * diff[b,n,t],
 *   diff[b,n,t]   = (output[b,n,t-1] - output[b,n,t]) / Ts,   output[.., -1] = 0,
 * with grad_output and output of shape [nBatch, nNeurons, T] and grad_delay of nNeurons
 * floats (overwritten).  Replaces the composition in _delayFunction.backward,
 * src/slayer.py:950-954: conv with [-1, 1]/Ts (convKernel, src/cuda/convKernels.h:10-35),
 * an elementwise product and torch.sum over batch and time.
 */
int slayer_b200_delay_grad(float *grad_delay, const float *grad_output, const float *output,
                           int64_t nBatch, int64_t nNeurons, int64_t T, float Ts, void *stream);

/*
 * SRM spike generation followed by an axonal delay, with the spikes written once, already
 * delayed: delayed = shift(getSpikes(u), d), d_n = trunc(shift_n / Ts), shift_n = shift_lut[n]
 * if shift_lut is not NULL (nNeurons values, rows are [nBatch, nNeurons]) else `shift`.  u is
 * updated in place as by slayer_b200_srm_get_spikes.  Same bits as that call followed by
 * slayer_b200_shift_lut / _scalar (getSpikes<float>, src/cuda/spikeKernels.h:54-60, then
 * shift<float>, src/cuda/shiftKernels.h:63-136).  When T % 4 == 0, T <= 2048 and the buffers are
 * 16-byte aligned the undelayed spikes never reach memory and s_scratch is not touched (it may
 * be NULL); otherwise s_scratch (rows * T floats) receives them and the two steps run one after
 * the other, or, if s_scratch is NULL, the call returns SLAYER_B200_EUNSUPPORTED.
 */
int slayer_b200_srm_get_spikes_delayed(float *delayed, float *s_scratch, float *u, const float *nu,
                                       const float *shift_lut, float shift,
                                       int64_t nBatch, int64_t nNeurons, int64_t nuSize, int64_t T,
                                       float theta, float Ts, void *stream);

/*
 * Bit-packed spike tensors.  A spike tensor holds two values, 0 and 1/Ts; packed, a row of T
 * samples is ceil(T / 32) uint32 words, bit i of word w = "sample 32 w + i is a spike" (bits
 * past T are zero): 1/32 of the bytes the fp32 form of the reference's interface moves
 * (getSpikesKernel writes fp32 samples, src/cuda/spikeKernels.h:18-27).  pack_spikes sets a bit
 * where s is non-zero; unpack_spikes writes `value` where a bit is set and 0 elsewhere.
 */
int slayer_b200_pack_spikes(uint32_t *bits, const float *s, int64_t rows, int64_t T, void *stream);
int slayer_b200_unpack_spikes(float *s, const uint32_t *bits, int64_t rows, int64_t T, float value, void *stream);

/*
 * slayer_b200_srm_get_spikes with the spikes written in the bit-packed form above (the updated
 * potential u is the same fp32 tensor).  Same spike positions and same u as getSpikes<float>(),
 * src/cuda/spikeKernels.h:9-38, :54-60; 8 + 1/8 instead of 12 bytes per element.  Needs
 * T % 4 == 0, u 16-byte aligned and nuSize <= 257; otherwise SLAYER_B200_EUNSUPPORTED (run
 * slayer_b200_srm_get_spikes and slayer_b200_pack_spikes instead).
 */
int slayer_b200_srm_get_spikes_packed(uint32_t *bits, float *u, const float *nu,
                                      int64_t rows, int64_t nuSize, int64_t T, float theta, void *stream);

/*
 * slayer_b200_conv on a bit-packed spike tensor: out = conv(unpack(bits, spike_value), filter),
 * the same bits as the two calls (conv<float>(), src/cuda/convKernels.h:10-35, applied to the
 * spike tensor as spikeLayer.psp does, src/slayer.py:130-142); 4 + 1/8 instead of 8 bytes per
 * element.  SLAYER_B200_EUNSUPPORTED for filters too long for the tiled kernel.
 */
int slayer_b200_conv_packed(float *out, const uint32_t *bits, const float *filter,
                            int64_t rows, int64_t T, int64_t K, float spike_value, float Ts, void *stream);

/*
 * Address events -> spike tensor, on the device: event e = (x[e], y[e], p[e], t[e] in ms)
 * lands at out[n[e], p, y, x, rint(t / samplingTime) - tStart] of a [N, C, H, W, T] tensor
 * (rint in double precision, half to even) if every index is inside it, and is dropped
 * otherwise.  n may be NULL (all events in sample 0) and y may be NULL (y = 0).  sum_mode = 0:
 * the element is set to 1 / samplingTime (`out` is updated in place, `base` is not read);
 * sum_mode != 0: the element becomes base[...] + 1 / samplingTime, once per bin however many
 * events share it (`base` holds the tensor's original values and must not be `out`; elements no
 * event touches are left as they are in `out`).  Events are int32 / float64 device arrays.
 * Replaces event.toSpikeTensor, src/spikeFileIO.py:66-144 (index rounding :95-97, bounds
 * :102-107 and :121-128, 'OR' :108-112, 'SUM' :113-117 - an indexed "+=" there, which adds once
 * per distinct index), including its time shift tSt (:82-93; drawn on the host and passed in).
 */
int slayer_b200_bin_events(float *out, const float *base, const int32_t *n, const int32_t *x, const int32_t *y,
                           const int32_t *p, const double *t, int64_t nEvents,
                           int64_t N, int64_t C, int64_t H, int64_t W, int64_t T,
                           double samplingTime, int64_t tStart, int sum_mode, void *stream);

/*
 * The same binning ('OR' mode) into a bit-packed spike tensor: `bits` holds ceil(T / 32) uint32
 * words per [n, p, y, x] row and must be zeroed (or hold earlier events) before the call; bits
 * are set with atomic OR.  Index rules as above (src/spikeFileIO.py:95-112).
 */
int slayer_b200_bin_events_packed(uint32_t *bits, const int32_t *n, const int32_t *x, const int32_t *y,
                                  const int32_t *p, const double *t, int64_t nEvents,
                                  int64_t N, int64_t C, int64_t H, int64_t W, int64_t T,
                                  double samplingTime, int64_t tStart, void *stream);

/*
 * Spike-count loss, value and gradient in one pass.  For output spikes s[rows, T] (rows = batch
 * x classes), a target region [start, stop) in time steps (resolved like a Python slice of a
 * row) and a desired spike count per row:
 *   c[row]   = float( (double(Ts * sum_{t in region} s[t]) - desired_count[row]) / (stop - start) * scale )
 *   e[t]     = conv(s outside the region, filter)[t] + (t in region ? c[row] : 0)
 *   row_sq[row] = sum_t e[t]^2 (double)           loss = Ts / 2 * sum(row_sq)   (left to the caller)
 *   grad[row, t] = corr(Ts * e, filter)[t]        = d loss / d s
 * conv / corr as slayer_b200_conv / _corr (same chains, x Ts).  Replaces spikeLoss.numSpikes,
 * src/spikeLoss.py:85-104 (host NumPy for the counts and masks, then psp and a tensor sum), and
 * the backward pass autograd derives from it (psp backward = corr, src/slayer.py:892).
 * SLAYER_B200_EUNSUPPORTED for rows too long for the kernel's shared memory.
 */
int slayer_b200_num_spikes_loss(float *grad, double *row_sq, const float *s, const float *desired_count,
                                const float *filter, int64_t rows, int64_t T, int64_t K,
                                int64_t start, int64_t stop, float Ts, float scale, void *stream);

/*
 * slayer_b200_srm_get_spikes without any memory allocation, for callers that cannot allocate
 * device memory: an application that has already given all device memory to its own pool, or
 * code that runs where entering the CUDA allocator is not allowed (another library's callback,
 * a process whose memory footprint has been frozen).  The regular entry point obtains a small
 * status buffer with cudaMalloc the first time a device is used; this one keeps its scratch -
 * one int per block of 32 rows: cleared when a warp starts the block, set to the number of
 * 64-step tiles when it finishes it, or to a negative code if a bounded wait for a load ran
 * out (slayer_b200_srm_get_spikes_noalloc_status reads it back) - in a fixed 256 KB array
 * inside the library image, resident on every GPU that loads the library until the process
 * exits.  Same arguments and results as slayer_b200_srm_get_spikes, restricted to
 *   - rows <= 2,097,152 (65536 blocks of 32 rows); more is rejected with SLAYER_B200_EUNSUPPORTED,
 *   - T % 4 == 0, s and u 16-byte aligned, nuSize <= 257 (else SLAYER_B200_EUNSUPPORTED).
 * The first call on each device resolves the array's device address and raises the
 * shared-memory limit of every variant of the kernel (one per length class of the refractory
 * kernel), which also loads their code; make that first call outside any stream capture and
 * before the memory footprint is frozen.  Later calls only launch.  The call itself
 * runs no cudaMalloc / cudaFree and no allocating library routine.  All calls share the one
 * array (each launch clears the entries it uses), so calls that overlap on the GPU - two
 * streams, two host threads - race on it: issue them on one stream or serialise them.
 * It has no counterpart in the reference.
 */
int slayer_b200_srm_get_spikes_noalloc(float *s, float *u, const float *nu,
                                       int64_t rows, int64_t nuSize, int64_t T,
                                       float theta, float Ts, void *stream);

/*
 * Outcome of the most recent slayer_b200_srm_get_spikes_noalloc launch on the current device,
 * read from that entry point's fixed array: 0 if every block of 32 rows of a [rows, T] launch
 * was walked to its end; SLAYER_B200_EDEVICE if some block was not (a bounded wait for a load
 * ran out, so s and u are only partly written), with the index of the first such block in
 * *first_bad_block (may be NULL; -1 when all is well).  Pass the rows and T of that launch.
 * Allocates nothing either: the entries are copied in pieces into a buffer on the caller's
 * stack.  The copy waits for the device, so call it after the work, not between launches,
 * and not while another noalloc launch is running (same array).  SLAYER_B200_EINVAL before
 * the first noalloc call on the device.  It has no counterpart in the reference.
 */
int slayer_b200_srm_get_spikes_noalloc_status(int64_t rows, int64_t T, int64_t *first_bad_block);

/*
 * Read and clear the device-side status word of the current device.  Kernels that wait on a
 * hardware barrier (bulk tensor copies) poll a bounded number of times; if a wait ever runs
 * out they record a non-zero code here and return instead of hanging.  *status_out is 0 when
 * nothing went wrong.  This call synchronises with the device (it copies the word back), so
 * it belongs after a batch of work, not between launches.  It has no counterpart in the
 * reference, whose kernels neither wait on anything nor report errors.
 */
int slayer_b200_device_status(int *status_out);

/*
 * Exercise the give-up branch of the kernels' bounded waits without losing a copy: a one-thread
 * kernel polls, `polls` times (1 .. 2^20), a barrier that nothing will complete, then records
 * in the device status word the code a lost bulk copy would leave (0x5101) and returns.  It
 * neither faults nor hangs; slayer_b200_device_status() afterwards reports and clears the code.
 * For tests and bring-up.  It has no counterpart in the reference.
 */
int slayer_b200_selftest_bounded_wait(int polls, void *stream);

/*
 * Enable (non-zero, the default) or disable the bulk-tensor-copy code path of the kernels
 * that have one (SRM getSpikes when T % 4 == 0 and buffers are 16-byte aligned); returns the
 * previous setting.  Disabled, those kernels use their cp.async path, which computes the same
 * results.  It has no counterpart in the reference.
 */
int slayer_b200_set_tma(int enable);

/*
 * Select the conv / corr kernel; returns the previous setting.  0: the scalar kernel.  1: the
 * packed kernel (two rows per lane, two-wide fp32 FMAs, zero skipping) with its tile size chosen
 * per launch; 2: the packed kernel with half-size tiles (two CTAs per SM) wherever they fit;
 * 3: the packed kernel with full-size tiles (one CTA per SM).  All compute the same bits.  It has
 * no counterpart in the reference.
 */
int slayer_b200_set_fir_packed(int enable);

/*
 * Select the form of the scalar conv / corr kernel; returns the previous setting.  1: warps
 * take the 16-sample segments of a CTA's tiles round robin across tile boundaries and hand tiles
 * over through split-phase shared-memory barriers (bounded waits; a wait that runs out records
 * 0x5102 in the device status word); 2 (the default): the same with a larger register budget
 * where two CTAs per SM still fit, and with per-row offsets inside the tiles when the arrays are
 * 16-byte aligned but their rows are not (T % 4 != 0), so that copies and stores are 16 instead
 * of 8 or 4 bytes wide; 3: as 2 without the row offsets; 4: as 2 with the loop over the groups
 * of four taps always in the form that is left where the groups end (by default only where that
 * form measured faster); 0: one
 * CTA-wide barrier per tile.  All compute the same bits.  It has no counterpart in the reference.
 */
int slayer_b200_set_fir_flow(int mode);

/*
 * Stages (tiles of 32 rows x 64 steps) that every warp of the bulk-tensor-copy SRM spike kernel
 * keeps in shared memory in launches too large to be resident at once: 2 .. 8; returns the
 * previous setting, and only that for a value outside the range.  Fewer stages per warp leave
 * room for more warps per SM.  The result does not depend on it.  The no-allocation entry point
 * is not affected.  It has no counterpart in the reference.
 */
int slayer_b200_set_srm_stages(int stages);

/*
 * Zero skipping in conv / corr / conv_packed; returns the previous setting.  A zero sample leaves
 * every sum it enters unchanged, so all settings give the same bits.
 *   0: never.
 *   1 (the default): conv and conv_packed inputs of at least 2^25 samples with rows of 64 .. 4096
 *      steps and at most 1024 taps are sampled by a probe kernel (corr, which filters gradients, is
 *      not); if at most 6 % (conv_packed: 9 %) of the sampled samples are non-zero
 *      (spike tensors) and every tap is finite, the event-driven kernel runs - a warp lists the
 *      non-zero samples of a row and adds their contributions to the outputs they reach, work in
 *      proportion to events x taps - otherwise the dense kernel.  The decision stays on the
 *      device: both kernels are enqueued and the one ruled out returns at once.  The packed
 *      two-row kernel (slayer_b200_set_fir_packed) also skips sample positions that are zero in
 *      all 64 rows of a tile.
 *   2: the event-driven kernel for every input it can take, whatever the density (testing).
 * The decision of a probed call lives in one of 64 slots of a per-device ring (1 KB, allocated by
 * the first probed call on the device: make that call outside stream capture).  Calls on one
 * stream never share a live slot; calls on different streams, or replays of graphs captured from
 * them, do once more than 64 probed calls lie between them - keep concurrent streams closer than
 * that, or switch the probe off (mode 0 or 2) for them.
 * It has no counterpart in the reference.
 */
int slayer_b200_set_fir_skip_zeros(int mode);

#ifdef __cplusplus
}
#endif
#endif /* SLAYER_B200_H_INCLUDED */
