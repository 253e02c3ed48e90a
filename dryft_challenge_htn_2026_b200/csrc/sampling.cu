// Token choice from float32 logits: greedy argmax (temperature 0; reference: engine/engine.py:503)
// and temperature sampling by the Gumbel-max rule, token = argmax_i(logit_i / T + g_i) with
// g_i = -log(-log(u_i)), u_i uniform in (0,1) from a counter hash of (seed, position, i). One pass
// over the row, no softmax normalisation, and the draw of a sequence depends only on its own seed
// and position, never on the batch it is in. Ties go to the lowest index.
#include "sampling_kernels.cuh"

DK_EXPORT int dk_sample_chunks(int V) { return (V + SAMPLE_CHUNK - 1) / SAMPLE_CHUNK; }

// logits [n_rows, V] float32; temperature [n_rows]; seeds [n_rows][2] (low, high word);
// ws_val / ws_idx: n_rows * dk_sample_chunks(V) elements of scratch.
DK_EXPORT int dk_sample(const float* logits, int n_rows, int V, const float* temperature, const uint32_t* seeds,
                        int* pos, const int* rows, float* ws_val, int* ws_idx, int* out_tok, int advance,
                        cudaStream_t st) {
    const int chunks = dk_sample_chunks(V);
    int e = dk_launch(sample_partial_kernel, dim3(chunks, n_rows), dim3(256), 0, st, logits, V, temperature, seeds,
                      (const int*)pos, rows, ws_val, ws_idx);
    if (e) return e;
    return dk_launch(sample_final_kernel, dim3(n_rows), dim3(32), 0, st, (const float*)ws_val, (const int*)ws_idx,
                     chunks, pos, rows, out_tok, advance);
}
