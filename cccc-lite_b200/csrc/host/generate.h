// The host side of token generation as cccc-llm drives it (cccc-llm/cccc-llm.cpp:181-577): the
// sampler over one row of logits and the prefill / decode / KV-rebuild loop, with the model behind
// a callback so that the same loop runs one GPU, tensor-parallel ranks, or (in the CPU tests) a
// table of canned logits.  Tokenising and the chat template stay with the caller, as token ids.
#pragma once

#include <functional>
#include <random>
#include <vector>

namespace cccc
{

// cccc-llm.cpp:113-118: defaults are greedy, no penalty.
struct SamplerConfig
{
    float temperature = 0.0f;           // <= 0: greedy arg-max (after bans and the repetition penalty)
    int top_k = 0;                      // 0: no top-k filter
    float top_p = 1.0f;                 // 1: no nucleus filter
    float repetition_penalty = 1.0f;    // applied to tokens seen in the last 512 context tokens
    std::vector<int> banned_ids;        // control tokens that must never be emitted
    bool needsLogits() const { return temperature > 0.0f || repetition_penalty != 1.0f || !banned_ids.empty(); }
};

// One token from V float logits: the algorithm of sample_logits (cccc-llm.cpp:181-343), step for step.
// `logits` is modified.  ctx_ids: the context so far (for the repetition penalty).
int sampleLogits(std::vector<float>& logits, const SamplerConfig& cfg, const std::vector<int>& ctx_ids, std::mt19937& rng);

struct GenerateConfig
{
    std::vector<int> eos_ids;
    int think_open_id = -1, think_close_id = -1;
    int sys_n = 0;       // leading tokens of ctx_ids that are the system prompt
    int turn_n = 0;      // tokens of the current user turn + assistant header that follow them
    int T = 0;           // most tokens one prefill takes (the reference's prefill net width)
    int T_kv = 0;        // KV-cache capacity in rows
    SamplerConfig sampler;
};

class Generator
{
public:
    // One decode step: feed `token` at cache row `pos`; return the arg-max token, and when
    // logits_out is not null also fill it with the V float logits of that step.
    using StepFn = std::function<int(int token, int pos, std::vector<float>* logits_out)>;
    // Clears the cache before a (re)prefill (Net::resetKVCache).
    using ResetFn = std::function<void()>;

    Generator(int vocab, StepFn step, ResetFn reset, unsigned int seed = 0) : V_(vocab), step_(std::move(step)), reset_(std::move(reset)), rng_(seed) {}

    // Generates up to max_new_tokens after ctx_ids (which it extends, and truncates on a KV rebuild exactly
    // as run_generate does, cccc-llm.cpp:347-577).  Returns the generated ids, EOS excluded.
    std::vector<int> generate(std::vector<int>& ctx_ids, const GenerateConfig& cfg, int max_new_tokens);

    int rebuilds() const { return rebuilds_; }
    int decodeSteps() const { return decode_steps_; }
    int prefillTokens() const { return prefill_tokens_; }

private:
    // Feeds tokens[0..n) at rows 0..n-1 and samples from the last one's logits.
    int prefill(const std::vector<int>& tokens, const GenerateConfig& cfg, const std::vector<int>& ctx_ids);
    int V_;
    StepFn step_;
    ResetFn reset_;
    std::mt19937 rng_;
    std::vector<float> logits_;
    int rebuilds_ = 0, decode_steps_ = 0, prefill_tokens_ = 0;
};

}    // namespace cccc
