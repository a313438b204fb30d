// The host side of greedy decoding, in native code: launch the captured step, wait for its tokens,
// feed them back, until a token needs a decision that belongs to the generation loop.
//
// The reference's loop samples on the host and calls the forward pass once per token
// (api/LLMEngine.java:743-769), replaying one captured graph per call (java21
// inference/CudaForwardPass.java:1760-1812). Here the captured graph holds, for a batch of sequences
// that each bring one token: the copy of the step's integers (tokens, positions, lengths) from
// page-locked host memory to the device, the model walk, the first-maximum argmax of every row, and
// the copy of the chosen tokens back to page-locked host memory. This loop runs that graph step after
// step without going back to the interpreter: every step still takes its input tokens from the host
// and returns its output tokens to the host.
//
// A step is *quiet* when every sequence simply goes on: no chosen token is one of the sequence's stop
// tokens, and no sequence has used up its budget of quiet steps (what is left of its token budget and
// of the context, as the generation loop computes it). The loop returns after the first step that is
// not quiet (its tokens are returned too, undecided), or after `max_steps`; the caller applies the
// generation loop's own rules to every returned token, so the rules live in one place.
#include "common.cuh"

// meta:      the page-locked image of the step's integers; tokens at [tokens_at, +B), positions at
//            [positions_at, +B), lengths at [lengths_at, +B) describe the NEXT step to run on entry, and
//            the last step that ran on return.
// sampled:   page-locked, [B]: where the graph's last node leaves the chosen tokens.
// quiet:     [B]: how many more chosen tokens of sequence i are certain to need no decision other than
//            "is it a stop token" (0: the next one already does).
// stop_ids / stop_begin: sequence i stops at stop_ids[stop_begin[i] .. stop_begin[i + 1]).
// out:       [max_steps, B]: the chosen tokens of every step that ran. steps_run: how many did.
extern "C" int lp_decode_loop(cudaGraphExec_t graph, cudaStream_t stream, int* meta, int tokens_at, int positions_at,
                              int lengths_at, const int* sampled, int B, int max_steps, const int* quiet,
                              const int* stop_ids, const int* stop_begin, int* out, int* steps_run) {
    *steps_run = 0;
    if (B <= 0 || max_steps <= 0) return 0;
    if (!graph || !meta || !sampled || !quiet || !stop_begin || !out) LP_REFUSE("decode_loop: a null argument");
    int fewest = quiet[0];
    for (int i = 1; i < B; ++i) fewest = quiet[i] < fewest ? quiet[i] : fewest;
    // The graph's last node copies the chosen tokens (all >= 0) into `sampled`. The loop marks the words with -1
    // before each launch and watches them turn: that sees the end of a step a few microseconds before the stream's
    // synchronisation wakes up. After a bounded number of looks it synchronises instead, and it always does so
    // before it returns.
    volatile int* fresh = const_cast<volatile int*>(sampled);
    for (int step = 0; step < max_steps; ++step) {
        for (int i = 0; i < B; ++i) fresh[i] = -1;
        cudaError_t err = cudaGraphLaunch(graph, stream);
        if (err == cudaSuccess) {
            bool seen = false;
            for (long spin = 0; spin < 2000000 && !seen; ++spin) {
                seen = true;
                for (int i = 0; i < B; ++i) seen = seen && fresh[i] >= 0;
            }
            if (!seen) err = cudaStreamSynchronize(stream);     // after it every word is set
        }
        if (err != cudaSuccess) {
            cudaStreamSynchronize(stream);
            snprintf(lp_error_text, sizeof(lp_error_text), "decode_loop: step %d: %s", step, cudaGetErrorString(err));
            return (int)err;
        }
        int* row = out + (size_t)step * B;
        bool goes_on = step < fewest;
        for (int i = 0; i < B; ++i) {
            const int tok = fresh[i];
            row[i] = tok;
            for (int s = stop_begin[i]; s < stop_begin[i + 1]; ++s) goes_on = goes_on && stop_ids[s] != tok;
        }
        *steps_run = step + 1;
        if (!goes_on || step + 1 == max_steps) break;
        for (int i = 0; i < B; ++i) {
            meta[tokens_at + i] = row[i];
            meta[positions_at + i] += 1;
            meta[lengths_at + i] += 1;
        }
    }
    cudaError_t err = cudaStreamSynchronize(stream);
    if (err != cudaSuccess) {
        snprintf(lp_error_text, sizeof(lp_error_text), "decode_loop: %s", cudaGetErrorString(err));
        return (int)err;
    }
    return 0;
}
