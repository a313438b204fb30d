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

// ---------------------------------------------------------------- the same loop with the sampler's draw
// For samplers whose state is a generator and a window of recent tokens (temperature, top-k, top-p, min-p and
// the repetition penalty of sampler/CompositeSampler.java:45-55, :387-395; not DRY, not mirostat): the captured
// graph also brings the step's sampler block from page-locked memory and runs the sampling kernels, and this
// loop keeps what the host keeps between two draws: java.util.Random's 48-bit state per sequence (one float per
// sampled token) and, per sequence, the distinct tokens among its recent ones in ascending order with the
// number of their occurrences (the penalty is multiplied up once per occurrence, in double, as the interpreter's
// sampler does).
//
// blob (page-locked, int32 words): B records of `record_words` words (the static fields are filled by the caller;
// this loop sets uniform, edit_begin, edit_count), then per sequence `cap` edit tokens, then `cap` amounts to
// subtract (always 0 here), then `cap` factors: edit arrays of sequence i begin at i * cap.
namespace {
struct Window {
    int* recent; int len, max_len;          // the tokens in order of arrival (oldest first)
    int* tok; int* cnt; int distinct;       // distinct tokens ascending, with their counts
};
inline int window_find(const Window& w, int token) {      // first index with tok >= token
    int lo = 0, hi = w.distinct;
    while (lo < hi) { const int mid = (lo + hi) >> 1; if (w.tok[mid] < token) lo = mid + 1; else hi = mid; }
    return lo;
}
inline void window_add(Window& w, int token) {
    const int at = window_find(w, token);
    if (at < w.distinct && w.tok[at] == token) { ++w.cnt[at]; return; }
    memmove(w.tok + at + 1, w.tok + at, sizeof(int) * (w.distinct - at));
    memmove(w.cnt + at + 1, w.cnt + at, sizeof(int) * (w.distinct - at));
    w.tok[at] = token; w.cnt[at] = 1; ++w.distinct;
}
inline void window_drop(Window& w, int token) {
    const int at = window_find(w, token);
    if (at >= w.distinct || w.tok[at] != token) return;
    if (--w.cnt[at] > 0) return;
    memmove(w.tok + at, w.tok + at + 1, sizeof(int) * (w.distinct - at - 1));
    memmove(w.cnt + at, w.cnt + at + 1, sizeof(int) * (w.distinct - at - 1));
    --w.distinct;
}
}  // namespace

// rng_state [B] (in/out), draws [B] (1: the sequence takes one float per token), penalty [B] (1.0: none),
// recent [B, cap] with recent_len [B] (in/out, oldest first) and window_len [B] (how many recent tokens sequence i
// keeps, at most cap), scratch [2 * B * cap] ints for this loop's tables.
// field_uniform / field_begin / field_count: word offsets of those fields in a record.
extern "C" int lp_decode_loop_sampled(cudaGraphExec_t graph, cudaStream_t stream, int* meta, int tokens_at,
                                      int positions_at, int lengths_at, int* blob, int record_words, int field_uniform,
                                      int field_begin, int field_count, int cap, const int* sampled, int B,
                                      int max_steps, const int* quiet, const int* stop_ids, const int* stop_begin,
                                      unsigned long long* rng_state, const int* draws, const double* penalty,
                                      int* recent, int* recent_len, const int* window_len, int* scratch, int* out,
                                      int* steps_run) {
    *steps_run = 0;
    if (B <= 0 || max_steps <= 0) return 0;
    if (!graph || !meta || !blob || !sampled || !quiet || !stop_begin || !out || !rng_state || !draws || !penalty ||
        !recent || !recent_len || !window_len || !scratch)
        LP_REFUSE("decode_loop_sampled: a null argument");
    if (B > 4096) LP_REFUSE("decode_loop_sampled: %d sequences", B);
    static Window windows[4096];
    for (int i = 0; i < B; ++i) {
        Window& w = windows[i];
        w.recent = recent + (size_t)i * cap; w.len = recent_len[i]; w.max_len = window_len[i];
        if (w.max_len < 1 || w.max_len > cap) LP_REFUSE("decode_loop_sampled: a window of %d tokens (capacity %d)", w.max_len, cap);
        w.tok = scratch + (size_t)i * cap; w.cnt = scratch + (size_t)(B + i) * cap; w.distinct = 0;
        if (w.len > w.max_len) LP_REFUSE("decode_loop_sampled: %d recent tokens for a window of %d", w.len, w.max_len);
        if (penalty[i] != 1.0) for (int j = 0; j < w.len; ++j) window_add(w, w.recent[j]);
    }
    int* edit_tok = blob + (size_t)B * record_words;
    float* edit_sub = reinterpret_cast<float*>(edit_tok + (size_t)B * cap);
    float* edit_fac = reinterpret_cast<float*>(edit_tok + (size_t)2 * B * cap);
    int fewest = quiet[0];
    for (int i = 1; i < B; ++i) fewest = quiet[i] < fewest ? quiet[i] : fewest;
    volatile int* fresh = const_cast<volatile int*>(sampled);
    int rc = 0;
    for (int step = 0; step < max_steps; ++step) {
        for (int i = 0; i < B; ++i) {
            int* rec = blob + (size_t)i * record_words;
            float uniform = 0.f;
            if (draws[i]) {
                rng_state[i] = (rng_state[i] * 0x5DEECE66DULL + 0xBULL) & ((1ULL << 48) - 1);
                uniform = (float)((double)(rng_state[i] >> 24) / 16777216.0);
            }
            memcpy(rec + field_uniform, &uniform, 4);
            const Window& w = windows[i];
            rec[field_begin] = i * cap;
            rec[field_count] = w.distinct;
            for (int j = 0; j < w.distinct; ++j) {
                double power = 1.0;
                for (int k = 0; k < w.cnt[j]; ++k) power *= penalty[i];
                edit_tok[(size_t)i * cap + j] = w.tok[j];
                edit_sub[(size_t)i * cap + j] = 0.f;
                edit_fac[(size_t)i * cap + j] = (float)power;
            }
            fresh[i] = -1;
        }
        cudaError_t err = cudaGraphLaunch(graph, stream);
        if (err == cudaSuccess) {
            bool seen = false;
            for (long spin = 0; spin < 2000000 && !seen; ++spin) {
                seen = true;
                for (int i = 0; i < B; ++i) seen = seen && fresh[i] >= 0;
            }
            if (!seen) err = cudaStreamSynchronize(stream);
        }
        if (err != cudaSuccess) {
            cudaStreamSynchronize(stream);
            snprintf(lp_error_text, sizeof(lp_error_text), "decode_loop_sampled: step %d: %s", step, cudaGetErrorString(err));
            rc = (int)err;
            break;
        }
        int* row = out + (size_t)step * B;
        bool goes_on = step < fewest;
        for (int i = 0; i < B; ++i) {
            const int tok = fresh[i];
            row[i] = tok;
            for (int s = stop_begin[i]; s < stop_begin[i + 1]; ++s) goes_on = goes_on && stop_ids[s] != tok;
            // the sampler takes the token in: the window moves on
            Window& w = windows[i];
            if (w.len == w.max_len) {
                if (penalty[i] != 1.0) window_drop(w, w.recent[0]);
                memmove(w.recent, w.recent + 1, sizeof(int) * (w.len - 1));
                --w.len;
            }
            w.recent[w.len++] = tok;
            if (penalty[i] != 1.0) window_add(w, tok);
        }
        *steps_run = step + 1;
        if (!goes_on || step + 1 == max_steps) break;
        for (int i = 0; i < B; ++i) {
            meta[tokens_at + i] = row[i];
            meta[positions_at + i] += 1;
            meta[lengths_at + i] += 1;
        }
    }
    for (int i = 0; i < B; ++i) recent_len[i] = windows[i].len;
    cudaError_t err = cudaStreamSynchronize(stream);
    if (rc == 0 && err != cudaSuccess) {
        snprintf(lp_error_text, sizeof(lp_error_text), "decode_loop_sampled: %s", cudaGetErrorString(err));
        rc = (int)err;
    }
    return rc;
}
