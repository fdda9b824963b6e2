// Reasoning-budget forcing of the step path (reference: budget_machine in
// crates/retrograd-ffi/runtime/src/retro_gen_core.cpp:890-1007, driven from the step at :2609-2680 and
// :2727-2760). The reference keeps the state machine inside llama.cpp's common library
// (common_reasoning_budget_*, a third-party dependency that is not part of its tree); this file restates that
// published machine:
//
//   IDLE      until one of the start tags has gone by token for token           -> COUNTING (budget 0: FORCING)
//   COUNTING  every accepted token costs one; an end tag going by means the model closed the block -> DONE;
//             the budget spent -> FORCING, or WAITING when the last token stopped inside a UTF-8 sequence
//   WAITING   tokens pass until one completes the sequence (or an end tag goes by)                   -> FORCING
//   FORCING   the forced tokens (the first end tag) are emitted one per accepted token               -> DONE
//
// The engine samples on the GPU; a machine that is FORCING when a row samples hands its token to the sampling
// kernel, which reports that token with its log-probabilities instead of the drawn one. Tags come from the
// caller's chat-template layer as token ids (this library renders no templates).
#pragma once

#include <algorithm>
#include <cstdint>
#include <functional>
#include <string>
#include <vector>

namespace rb200 {

struct ReasoningPlan {
    bool active = false;
    int32_t budget = -1;                          // -1: the model decides
    std::vector<std::vector<int32_t>> starts;     // opening tags
    std::vector<std::vector<int32_t>> ends;       // closing tags; the first is the one a spent budget forces
    std::vector<int32_t> forced;
    size_t n_prompt_tail = 0;                     // how much of a prompt's end is replayed into a fresh machine
    bool operator==(const ReasoningPlan & o) const {
        return active == o.active && budget == o.budget && starts == o.starts && ends == o.ends && forced == o.forced &&
               n_prompt_tail == o.n_prompt_tail;
    }
};

class BudgetMachine {
public:
    enum State { IDLE, COUNTING, WAITING_UTF8, FORCING, DONE };

    BudgetMachine() = default;
    // `complete`: whether a token's text ends on a UTF-8 character boundary
    BudgetMachine(const ReasoningPlan * plan, std::function<bool(int32_t)> complete) : plan_(plan && plan->active ? plan : nullptr), complete_(std::move(complete)) {
        if (plan_) {
            start_at_.assign(plan_->starts.size(), 0);
            end_at_.assign(plan_->ends.size(), 0);
        }
    }

    bool active() const { return plan_ != nullptr; }
    State state() const { return state_; }
    // the token the machine is about to force, or -1
    int32_t pending() const { return plan_ && state_ == FORCING && force_pos_ < plan_->forced.size() ? plan_->forced[force_pos_] : -1; }

    void accept(int32_t token) {
        if (!plan_) return;
        switch (state_) {
            case IDLE:
                if (advance(plan_->starts, start_at_, token)) {
                    remaining_ = plan_->budget;
                    state_ = COUNTING;
                    if (remaining_ <= 0) begin_forcing();
                }
                break;
            case COUNTING:
            case WAITING_UTF8: {
                if (advance(plan_->ends, end_at_, token)) {
                    state_ = DONE;
                    break;
                }
                const bool whole = !complete_ || complete_(token);
                if (state_ == WAITING_UTF8) {
                    if (whole) begin_forcing();
                } else if (--remaining_ <= 0) {
                    if (whole) begin_forcing();
                    else state_ = WAITING_UTF8;
                }
                break;
            }
            case FORCING:
                if (++force_pos_ >= plan_->forced.size()) state_ = DONE;
                break;
            case DONE:
                break;
        }
    }

    // Replays the end of the prompt (retro_gen_core.cpp:952-975): a prompt that already opened the block starts the
    // machine counting, one that closed it starts it done. A machine that starts forcing on a prompt token stops
    // the replay there, unless the rest of the prompt closes the block itself: then the forced sequence is accepted
    // in its place and the replay resumes behind the tag.
    void prime(const int32_t * prompt, size_t n_prompt) {
        if (!plan_ || n_prompt == 0) return;
        const int32_t * end = prompt + n_prompt;
        const int32_t * at = prompt + (n_prompt - std::min(plan_->n_prompt_tail, n_prompt));
        while (at != end) {
            accept(*at++);
            if (state_ != FORCING) continue;
            const int32_t * closed = nullptr;
            const int32_t * earliest = end;
            for (const auto & tag : plan_->ends) {
                const int32_t * found = std::search(at, end, tag.begin(), tag.end());
                if (found != end && found < earliest) {
                    earliest = found;
                    closed = found + tag.size();
                }
            }
            if (!closed) return;
            for (const int32_t token : plan_->forced) accept(token);
            at = closed;
        }
    }

    // The token to emit in place of `sampled`, and whether the budget forced it (retro_gen_core.cpp:979-1005).
    int32_t next(int32_t sampled, bool & forced) {
        forced = false;
        if (!plan_) return sampled;
        int32_t token = sampled;
        if (state_ == FORCING && force_pos_ < plan_->forced.size()) {
            token = plan_->forced[force_pos_];
            forced = true;
        }
        accept(token);
        return token;
    }

private:
    // every tag is matched on its own: a token that breaks a partial match may start it again
    static bool advance(const std::vector<std::vector<int32_t>> & tags, std::vector<size_t> & at, int32_t token) {
        bool matched = false;
        for (size_t i = 0; i < tags.size(); ++i) {
            const std::vector<int32_t> & tag = tags[i];
            if (tag.empty()) continue;
            if (token == tag[at[i]]) {
                if (++at[i] >= tag.size()) {
                    at[i] = 0;
                    matched = true;
                }
            } else {
                at[i] = token == tag[0] ? 1 : 0;
                if (at[i] >= tag.size()) {
                    at[i] = 0;
                    matched = true;
                }
            }
        }
        if (matched) std::fill(at.begin(), at.end(), 0);
        return matched;
    }
    void begin_forcing() {
        state_ = FORCING;
        force_pos_ = 0;
        std::fill(end_at_.begin(), end_at_.end(), 0);
        if (plan_->forced.empty()) state_ = DONE;
    }

    const ReasoningPlan * plan_ = nullptr;
    std::function<bool(int32_t)> complete_;
    State state_ = IDLE;
    int32_t remaining_ = 0;
    size_t force_pos_ = 0;
    std::vector<size_t> start_at_, end_at_;
};

// Whether `text` ends on a UTF-8 character boundary.
inline bool utf8_is_complete(const std::string & text) {
    size_t i = text.size(), tail = 0;
    while (i > 0 && tail < 4 && (static_cast<unsigned char>(text[i - 1]) & 0xC0) == 0x80) {
        --i;
        ++tail;
    }
    if (i == 0) return tail == 0;
    const unsigned char lead = static_cast<unsigned char>(text[i - 1]);
    const size_t want = lead < 0x80 ? 0 : (lead >> 5) == 0x6 ? 1 : (lead >> 4) == 0xE ? 2 : (lead >> 3) == 0x1E ? 3 : tail;
    return tail == want;
}

} // namespace rb200
