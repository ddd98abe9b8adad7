/* Measurement and checker hooks of libbitnet_b200.so.  Not part of the drop-in boundary: the
 * benchmark and the tests use them; a deployment does not need this header. */
#ifndef BITNET_B200_BENCH_H
#define BITNET_B200_BENCH_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Enqueues only the four BitLinear kernels of every layer of a decoder (no attention, no
 * output head), so that the BitLinear kernel can be timed alone on the model's real weights.
 * The activations it leaves behind are meaningless. */
int bitnet_decoder_bench_linears(void* decoder, int64_t* tokens, void* stream);
/* Makes every attention kernel of the decoder's step also store its bf16 output to
 * buffer[layer][batch][dim] (NULL switches it off), so that a checker can follow the step with
 * the very same attention outputs.  Takes effect for steps enqueued (or captured) afterwards. */
int bitnet_decoder_set_attention_tap(void* decoder, void* buffer);
/* In a library built with -DBITNET_TRACE, CTA 0 of every BitLinear launch of a decoder records
 * six %globaltimer stamps (start, weights requested, dependency resolved, activations quantised,
 * matmul done, results stored); this copies them out, sixteen 64-bit values per launch (the 4
 * BitLinear launches of every layer).  BITNET_STATUS_UNSUPPORTED in a regular build. */
int bitnet_decoder_read_trace(void* decoder, unsigned long long* host_out, int n_values);

#ifdef __cplusplus
}
#endif
#endif /* BITNET_B200_BENCH_H */
