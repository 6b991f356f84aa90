#include "generate.h"

#include <algorithm>
#include <cmath>
#include <cstdio>

namespace cccc
{

int sampleLogits(std::vector<float>& logits, const SamplerConfig& cfg, const std::vector<int>& ctx_ids, std::mt19937& rng)
{
    const int V = (int)logits.size();
    // control tokens never come out as text (cccc-llm.cpp:216-223)
    for (int id : cfg.banned_ids)
    {
        if (id >= 0 && id < V) { logits[id] = -1e30f; }
    }
    // repetition penalty over the last 512 context tokens (:225-245)
    if (cfg.repetition_penalty != 1.0f && !ctx_ids.empty())
    {
        const int start = (int)ctx_ids.size() > 512 ? (int)ctx_ids.size() - 512 : 0;
        for (int i = start; i < (int)ctx_ids.size(); i++)
        {
            const int id = ctx_ids[i];
            if (id >= 0 && id < V)
            {
                if (logits[id] > 0.0f) { logits[id] /= cfg.repetition_penalty; }
                else { logits[id] *= cfg.repetition_penalty; }
            }
        }
    }
    if (cfg.temperature <= 0.0f) { return (int)(std::max_element(logits.begin(), logits.end()) - logits.begin()); }    // :247-251
    for (auto& l : logits) { l /= cfg.temperature; }
    // top-k: everything below the k-th largest is removed (:259-272)
    if (cfg.top_k > 0 && cfg.top_k < V)
    {
        std::vector<float> tmp(logits.begin(), logits.end());
        std::nth_element(tmp.begin(), tmp.begin() + cfg.top_k - 1, tmp.end(), std::greater<float>());
        const float threshold = tmp[cfg.top_k - 1];
        for (auto& l : logits)
        {
            if (l < threshold) { l = -1e30f; }
        }
    }
    // softmax (:274-288)
    const float max_l = *std::max_element(logits.begin(), logits.end());
    float sum = 0.0f;
    for (auto& l : logits)
    {
        l = std::exp(l - max_l);
        sum += l;
    }
    if (sum > 0.0f)
    {
        for (auto& l : logits) { l /= sum; }
    }
    // nucleus: tokens after the cumulative probability passes top_p are dropped (:290-325)
    if (cfg.top_p < 1.0f)
    {
        std::vector<std::pair<float, int>> sp(V);
        for (int i = 0; i < V; i++) { sp[i] = { logits[i], i }; }
        std::sort(sp.begin(), sp.end(), std::greater<std::pair<float, int>>());
        float cum = 0.0f;
        bool cutting = false;
        for (auto& pi : sp)
        {
            if (cutting)
            {
                logits[pi.second] = 0.0f;
                continue;
            }
            cum += pi.first;
            if (cum > cfg.top_p) { cutting = true; }
        }
        sum = 0.0f;
        for (auto& l : logits) { sum += l; }
        if (sum > 0.0f)
        {
            for (auto& l : logits) { l /= sum; }
        }
    }
    // multinomial draw (:327-342)
    std::uniform_real_distribution<float> dist(0.0f, 1.0f);
    const float r = dist(rng);
    float cum = 0.0f;
    for (int i = 0; i < V; i++)
    {
        cum += logits[i];
        if (r <= cum) { return i; }
    }
    return V - 1;
}

int Generator::prefill(const std::vector<int>& tokens, const GenerateConfig& cfg, const std::vector<int>& ctx_ids)
{
    // The reference prefills all rows in one pass of its prefill net; here the rows go through the decode step
    // one after the other, which fills the same cache rows and ends with the same last-row logits.
    reset_();
    const bool want = cfg.sampler.needsLogits();
    int next = 0;
    for (size_t i = 0; i < tokens.size(); i++)
    {
        const bool last = i + 1 == tokens.size();
        next = step_(tokens[i], (int)i, (last && want) ? &logits_ : nullptr);
        prefill_tokens_++;
    }
    if (want && !tokens.empty()) { next = sampleLogits(logits_, cfg.sampler, ctx_ids, rng_); }
    return next;
}

std::vector<int> Generator::generate(std::vector<int>& ctx_ids, const GenerateConfig& cfg, int max_new_tokens)
{
    std::vector<int> out;
    if (ctx_ids.empty() || cfg.T <= 0) { return out; }
    // ---- prefill: the last n <= T tokens of the context (cccc-llm.cpp:355-391) ----
    const int n = std::min((int)ctx_ids.size(), cfg.T);
    const int offset = (int)ctx_ids.size() - n;
    int next_id = prefill(std::vector<int>(ctx_ids.begin() + offset, ctx_ids.end()), cfg, ctx_ids);
    int pos = n;
    int ctx_at_start = (int)ctx_ids.size();
    int think_depth = 0;
    for (int step = 0; step < max_new_tokens; step++)
    {
        if (std::find(cfg.eos_ids.begin(), cfg.eos_ids.end(), next_id) != cfg.eos_ids.end()) { break; }
        ctx_ids.push_back(next_id);
        out.push_back(next_id);
        if (cfg.think_open_id >= 0 && next_id == cfg.think_open_id) { think_depth++; }
        else if (cfg.think_close_id >= 0 && next_id == cfg.think_close_id && think_depth > 0) { think_depth--; }
        // ---- the cache is full: re-prefill [system | current turn | tail] (cccc-llm.cpp:439-533) ----
        if (cfg.T_kv > 0 && pos >= cfg.T_kv)
        {
            if (++rebuilds_ > 4)
            {
                std::fprintf(stderr, "[llm] KV-cache rebuild limit reached, stopping.\n");
                break;
            }
            const int sys_n = cfg.sys_n, turn_n = cfg.turn_n;
            const int anchor_n = sys_n + turn_n;
            const int gen_so_far = (int)ctx_ids.size() - ctx_at_start;
            int max_rebuild = std::min(cfg.T, cfg.T_kv / 2);
            if (max_rebuild <= anchor_n) { max_rebuild = anchor_n + 1; }
            const int max_tail = max_rebuild - anchor_n;
            // the reference fills a zeroed buffer of T ids at fixed indices (:462-476); the same indices here
            int tail_n = 0;
            std::vector<int> x((size_t)std::max(cfg.T, max_rebuild + 1), 0);
            for (int i = 0; i < sys_n && i < cfg.T; i++) { x[i] = ctx_ids[i]; }
            for (int i = 0; i < turn_n && sys_n + i < cfg.T; i++) { x[sys_n + i] = ctx_ids[sys_n + i]; }
            if (think_depth > 0 && cfg.think_open_id >= 0)
            {
                // still thinking: the marker, then the newest generated tokens (:480-491)
                x[anchor_n] = cfg.think_open_id;
                const int actual_tail = std::min(gen_so_far, max_tail - 1);
                const int start = (int)ctx_ids.size() - actual_tail;
                for (int i = 0; i < actual_tail; i++) { x[anchor_n + 1 + i] = ctx_ids[start + i]; }
                tail_n = 1 + actual_tail;
            }
            else
            {
                // not thinking: the newest tokens from before this generation started, so that earlier
                // tool results survive; the tail ends at the assistant header (:493-510)
                const int available = ctx_at_start - anchor_n;
                const int actual_tail = std::max(0, std::min(available, max_tail));
                const int start = ctx_at_start - actual_tail;
                for (int i = 0; i < actual_tail; i++) { x[anchor_n + i] = ctx_ids[start + i]; }
                tail_n = actual_tail;
            }
            const int rebuild_n = anchor_n + tail_n;
            x.resize((size_t)rebuild_n);
            // sampled with the context as it is before the cut, then the context is cut to rebuild_n entries:
            // the reference truncates ctx_ids (resize, :524-529), it does not copy the rebuilt row into it
            next_id = prefill(x, cfg, ctx_ids);
            ctx_ids.resize((size_t)rebuild_n);
            pos = rebuild_n;
            ctx_at_start = rebuild_n;
            continue;
        }
        // ---- one decode step at row pos (cccc-llm.cpp:536-548) ----
        const bool want = cfg.sampler.needsLogits();
        next_id = step_(next_id, pos, want ? &logits_ : nullptr);
        if (want) { next_id = sampleLogits(logits_, cfg.sampler, ctx_ids, rng_); }
        pos++;
        decode_steps_++;
    }
    return out;
}

}    // namespace cccc
