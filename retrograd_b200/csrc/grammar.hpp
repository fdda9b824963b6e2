// GBNF grammars for constrained sampling, host side.
//
// The reference compiles a row's GBNF text with its llama.cpp fork and asks the compiled sampler, before every
// draw, which tokens may come next (crates/retrograd-ffi/runtime/src/retro_gen_core.cpp:2518-2537 compile,
// :773-798 mask, :2738-2745 accept; the transformation order bias -> penalties -> GRAMMAR MASK -> top_k -> ... is
// pinned in retro_lora_train.h:1364-1369). The fork is not part of the reference checkout, so this is a
// grammar engine of this library's own for the published GBNF notation: rules `name ::= ...`, alternatives `|`,
// literals "..." (escapes \n \t \r \\ \" \[ \] \xHH \uHHHH \UHHHHHHHH), character classes [a-z0-9_] and [^...],
// `.` for any character, groups ( ... ), the repetitions * + ? {m} {m,} {m,n}, `#` comments. The start rule is
// `root`. Matching is a pushdown automaton over Unicode code points kept as a set of stacks; the step path
// turns the set into a per-token bit mask on the host (it does not depend on the logits), the sampling kernel
// applies it, and the sampled token advances the set.
#pragma once

#include <algorithm>
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace rb200 {

class Grammar {
public:
    struct Symbol {
        int32_t rule = -1;                                  // >= 0: a reference to that rule; -1: a character set
        bool negated = false, any = false;
        std::vector<std::pair<uint32_t, uint32_t>> ranges;  // inclusive code point ranges
        bool matches(uint32_t c) const {
            if (any) return true;
            bool in = false;
            for (const auto & r : ranges)
                if (c >= r.first && c <= r.second) { in = true; break; }
            return in != negated;
        }
    };
    using Alternative = std::vector<Symbol>;
    struct Pos { int32_t rule, alt, idx; bool operator==(const Pos & o) const { return rule == o.rule && alt == o.alt && idx == o.idx; }
                 bool operator<(const Pos & o) const { return rule != o.rule ? rule < o.rule : alt != o.alt ? alt < o.alt : idx < o.idx; } };
    using Stack = std::vector<Pos>;        // the position to match next is at the back; an empty stack = the grammar is complete

    // Throws std::invalid_argument on a malformed grammar, a missing rule, a missing `root` or left recursion.
    explicit Grammar(const std::string & text) {
        Parser(*this, text).run();
        auto root = names_.find("root");
        if (root == names_.end() || rules_[root->second].empty()) throw std::invalid_argument("the grammar has no root rule");
        root_ = root->second;
        for (size_t r = 0; r < rules_.size(); ++r)
            if (rules_[r].empty()) throw std::invalid_argument("the grammar references an undefined rule");
        reject_left_recursion();
    }

    std::vector<Stack> initial() const {
        std::vector<Stack> out;
        for (int32_t a = 0; a < (int32_t)rules_[root_].size(); ++a) {
            Stack s;
            if (!rules_[root_][a].empty()) s.push_back(Pos{root_, a, 0});
            advance(s, out);
        }
        normalise(out);
        return out;
    }

    // The stacks after one more code point; empty when no stack accepts it.
    std::vector<Stack> accept(const std::vector<Stack> & stacks, uint32_t c) const {
        std::vector<Stack> out;
        for (const Stack & s : stacks) {
            if (s.empty()) continue;
            const Pos top = s.back();
            if (!symbol(top).matches(c)) continue;
            Stack next(s.begin(), s.end() - 1);
            if (top.idx + 1 < (int32_t)rules_[top.rule][top.alt].size()) next.push_back(Pos{top.rule, top.alt, top.idx + 1});
            advance(next, out);
        }
        normalise(out);
        return out;
    }

    static bool complete(const std::vector<Stack> & stacks) {
        for (const Stack & s : stacks)
            if (s.empty()) return true;
        return false;
    }

    bool first_matches(const std::vector<Stack> & stacks, uint32_t c) const {
        for (const Stack & s : stacks)
            if (!s.empty() && symbol(s.back()).matches(c)) return true;
        return false;
    }
    // Whether some stack could take a code point of at least 0x80 next (the continuation of an unfinished UTF-8 sequence).
    bool may_take_non_ascii(const std::vector<Stack> & stacks) const {
        for (const Stack & s : stacks) {
            if (s.empty()) continue;
            const Symbol & sym = symbol(s.back());
            if (sym.any || sym.negated) return true;
            for (const auto & r : sym.ranges)
                if (r.second >= 0x80) return true;
        }
        return false;
    }

private:
    std::vector<std::vector<Alternative>> rules_;
    std::unordered_map<std::string, int32_t> names_;
    int32_t root_ = 0;

    const Symbol & symbol(const Pos & p) const { return rules_[p.rule][p.alt][p.idx]; }

    // Expands rule references at the top of `s` until a character set (or nothing) is on top.
    void advance(const Stack & s, std::vector<Stack> & out) const {
        if (s.empty() || symbol(s.back()).rule < 0) {
            out.push_back(s);
            return;
        }
        const Pos top = s.back();
        const int32_t ref = symbol(top).rule;
        for (int32_t a = 0; a < (int32_t)rules_[ref].size(); ++a) {
            Stack next(s.begin(), s.end() - 1);
            if (top.idx + 1 < (int32_t)rules_[top.rule][top.alt].size()) next.push_back(Pos{top.rule, top.alt, top.idx + 1});
            if (!rules_[ref][a].empty()) next.push_back(Pos{ref, a, 0});
            advance(next, out);
        }
    }
    static void normalise(std::vector<Stack> & stacks) {
        std::sort(stacks.begin(), stacks.end());
        stacks.erase(std::unique(stacks.begin(), stacks.end()), stacks.end());
    }

    int32_t rule_id(const std::string & name) {
        auto found = names_.find(name);
        if (found != names_.end()) return found->second;
        rules_.emplace_back();
        names_[name] = (int32_t)rules_.size() - 1;
        return (int32_t)rules_.size() - 1;
    }
    int32_t fresh_rule() {
        rules_.emplace_back();
        return (int32_t)rules_.size() - 1;
    }

    // A rule that can derive the empty string, then: does some rule reach itself as its own leftmost symbol?
    void reject_left_recursion() const {
        const size_t n = rules_.size();
        std::vector<char> nullable(n, 0);
        for (bool changed = true; changed;) {
            changed = false;
            for (size_t r = 0; r < n; ++r) {
                if (nullable[r]) continue;
                for (const Alternative & alt : rules_[r]) {
                    bool all = true;
                    for (const Symbol & s : alt)
                        if (s.rule < 0 || !nullable[s.rule]) { all = false; break; }
                    if (all) { nullable[r] = 1; changed = true; break; }
                }
            }
        }
        std::vector<std::vector<int32_t>> leftmost(n);
        for (size_t r = 0; r < n; ++r)
            for (const Alternative & alt : rules_[r])
                for (const Symbol & s : alt) {
                    if (s.rule < 0) break;
                    leftmost[r].push_back(s.rule);
                    if (!nullable[s.rule]) break;
                }
        std::vector<char> state(n, 0);      // 0 unseen, 1 on the path, 2 done
        std::vector<std::pair<int32_t, size_t>> path;
        for (size_t start = 0; start < n; ++start) {
            if (state[start]) continue;
            path.push_back({(int32_t)start, 0});
            state[start] = 1;
            while (!path.empty()) {
                auto & [r, i] = path.back();
                if (i == leftmost[r].size()) {
                    state[r] = 2;
                    path.pop_back();
                    continue;
                }
                const int32_t next = leftmost[r][i++];
                if (state[next] == 1) throw std::invalid_argument("the grammar is left-recursive");
                if (state[next] == 0) {
                    state[next] = 1;
                    path.push_back({next, 0});
                }
            }
        }
    }

    class Parser {
    public:
        Parser(Grammar & g, const std::string & text) : g_(g), s_(text) {}
        void run() {
            skip_space(true);
            while (pos_ < s_.size()) {
                const std::string name = parse_name();
                skip_space(false);
                if (s_.compare(pos_, 3, "::=") != 0) fail("expected ::=");
                pos_ += 3;
                skip_space(true);
                const int32_t rule = g_.rule_id(name);
                if (!g_.rules_[rule].empty()) fail("a rule is defined twice");
                std::vector<Alternative> alts = parse_alternatives(false);
                g_.rules_[rule] = std::move(alts);
                skip_space(true);
            }
        }

    private:
        Grammar & g_;
        const std::string & s_;
        size_t pos_ = 0;

        [[noreturn]] void fail(const char * what) const { throw std::invalid_argument(std::string("invalid GBNF: ") + what + " at offset " + std::to_string(pos_)); }
        static bool name_char(char c) { return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z') || (c >= '0' && c <= '9') || c == '-' || c == '_'; }

        void skip_space(bool newline_ok) {
            while (pos_ < s_.size()) {
                const char c = s_[pos_];
                if (c == ' ' || c == '\t') ++pos_;
                else if (c == '#') { while (pos_ < s_.size() && s_[pos_] != '\n' && s_[pos_] != '\r') ++pos_; }
                else if ((c == '\n' || c == '\r') && newline_ok) ++pos_;
                else break;
            }
        }
        std::string parse_name() {
            const size_t start = pos_;
            while (pos_ < s_.size() && name_char(s_[pos_])) ++pos_;
            if (pos_ == start) fail("expected a rule name");
            return s_.substr(start, pos_ - start);
        }
        uint32_t hex(int digits) {
            uint32_t v = 0;
            for (int i = 0; i < digits; ++i, ++pos_) {
                if (pos_ >= s_.size()) fail("unfinished escape");
                const char c = s_[pos_];
                v <<= 4;
                if (c >= '0' && c <= '9') v |= (uint32_t)(c - '0');
                else if (c >= 'a' && c <= 'f') v |= (uint32_t)(c - 'a' + 10);
                else if (c >= 'A' && c <= 'F') v |= (uint32_t)(c - 'A' + 10);
                else fail("bad hex digit");
            }
            return v;
        }
        // One (possibly escaped, possibly multi-byte) character of a literal or a class.
        uint32_t parse_char() {
            if (pos_ >= s_.size()) fail("unexpected end");
            const unsigned char c = (unsigned char)s_[pos_];
            if (c == '\\') {
                if (pos_ + 1 >= s_.size()) fail("unfinished escape");
                const char e = s_[pos_ + 1];
                pos_ += 2;
                switch (e) {
                    case 'x': return hex(2);
                    case 'u': return hex(4);
                    case 'U': return hex(8);
                    case 't': return '\t';
                    case 'r': return '\r';
                    case 'n': return '\n';
                    case '\\': case '"': case '[': case ']': return (uint32_t)e;
                    default: fail("unknown escape");
                }
            }
            int extra = c >= 0xF0 ? 3 : c >= 0xE0 ? 2 : c >= 0xC0 ? 1 : 0;
            uint32_t cp = extra == 3 ? c & 0x07 : extra == 2 ? c & 0x0F : extra == 1 ? c & 0x1F : c;
            ++pos_;
            for (; extra > 0; --extra, ++pos_) {
                if (pos_ >= s_.size() || ((unsigned char)s_[pos_] & 0xC0) != 0x80) fail("bad UTF-8");
                cp = (cp << 6) | ((unsigned char)s_[pos_] & 0x3F);
            }
            return cp;
        }
        std::vector<Alternative> parse_alternatives(bool nested) {
            std::vector<Alternative> alts;
            alts.push_back(parse_sequence(nested));
            while (pos_ < s_.size() && s_[pos_] == '|') {
                ++pos_;
                skip_space(true);
                alts.push_back(parse_sequence(nested));
            }
            return alts;
        }
        Alternative parse_sequence(bool nested) {
            Alternative seq;
            size_t last = 0;            // where the symbols of the last item begin
            while (pos_ < s_.size()) {
                const char c = s_[pos_];
                if (c == '"') {
                    ++pos_;
                    last = seq.size();
                    while (pos_ < s_.size() && s_[pos_] != '"') {
                        Symbol sym;
                        const uint32_t cp = parse_char();
                        sym.ranges.push_back({cp, cp});
                        seq.push_back(std::move(sym));
                    }
                    if (pos_ >= s_.size()) fail("unterminated literal");
                    ++pos_;
                    skip_space(nested);
                } else if (c == '[') {
                    ++pos_;
                    Symbol sym;
                    if (pos_ < s_.size() && s_[pos_] == '^') { sym.negated = true; ++pos_; }
                    while (pos_ < s_.size() && s_[pos_] != ']') {
                        const uint32_t lo = parse_char();
                        uint32_t hi = lo;
                        if (pos_ + 1 < s_.size() && s_[pos_] == '-' && s_[pos_ + 1] != ']') {
                            ++pos_;
                            hi = parse_char();
                        }
                        sym.ranges.push_back({lo, hi});
                    }
                    if (pos_ >= s_.size()) fail("unterminated character class");
                    ++pos_;
                    last = seq.size();
                    seq.push_back(std::move(sym));
                    skip_space(nested);
                } else if (c == '.') {
                    ++pos_;
                    Symbol sym;
                    sym.any = true;
                    last = seq.size();
                    seq.push_back(std::move(sym));
                    skip_space(nested);
                } else if (name_char(c)) {
                    const std::string name = parse_name();
                    Symbol sym;
                    sym.rule = g_.rule_id(name);
                    last = seq.size();
                    seq.push_back(std::move(sym));
                    skip_space(nested);
                } else if (c == '(') {
                    ++pos_;
                    skip_space(true);
                    const int32_t sub = g_.fresh_rule();
                    std::vector<Alternative> alts = parse_alternatives(true);
                    g_.rules_[sub] = std::move(alts);
                    if (pos_ >= s_.size() || s_[pos_] != ')') fail("expected )");
                    ++pos_;
                    Symbol sym;
                    sym.rule = sub;
                    last = seq.size();
                    seq.push_back(std::move(sym));
                    skip_space(nested);
                } else if (c == '*' || c == '+' || c == '?' || c == '{') {
                    if (last >= seq.size()) fail("a repetition needs something to repeat");
                    long lo = 0, hi = -1;        // hi < 0: unbounded
                    if (c == '*') { ++pos_; }
                    else if (c == '+') { lo = 1; ++pos_; }
                    else if (c == '?') { hi = 1; ++pos_; }
                    else {
                        ++pos_;
                        skip_space(nested);
                        lo = parse_int();
                        hi = lo;
                        skip_space(nested);
                        if (pos_ < s_.size() && s_[pos_] == ',') {
                            ++pos_;
                            skip_space(nested);
                            hi = pos_ < s_.size() && s_[pos_] >= '0' && s_[pos_] <= '9' ? parse_int() : -1;
                            skip_space(nested);
                        }
                        if (pos_ >= s_.size() || s_[pos_] != '}') fail("expected }");
                        ++pos_;
                        if (hi >= 0 && hi < lo) fail("a repetition's upper bound is below its lower bound");
                        if (lo > 1000 || hi > 1000) fail("a repetition count above 1000");
                    }
                    repeat(seq, last, lo, hi);
                    last = seq.size();
                    skip_space(nested);
                } else {
                    break;
                }
            }
            return seq;
        }
        long parse_int() {
            if (pos_ >= s_.size() || s_[pos_] < '0' || s_[pos_] > '9') fail("expected a number");
            long v = 0;
            while (pos_ < s_.size() && s_[pos_] >= '0' && s_[pos_] <= '9' && v < 100000) v = v * 10 + (s_[pos_++] - '0');
            return v;
        }
        // Rewrites seq[last..] =: S as lo copies of S followed by (hi < 0: S*) or (hi - lo nested optional copies).
        void repeat(Alternative & seq, size_t last, long lo, long hi) {
            const Alternative item(seq.begin() + (long)last, seq.end());
            seq.resize(last);
            for (long i = 0; i < lo; ++i) seq.insert(seq.end(), item.begin(), item.end());
            if (hi < 0) {
                const int32_t star = g_.fresh_rule();        // star ::= S star | (nothing)
                Alternative again = item;
                Symbol self;
                self.rule = star;
                again.push_back(self);
                g_.rules_[star] = {again, Alternative{}};
                seq.push_back(self);
            } else {
                int32_t inner = -1;                          // opt_k ::= S opt_(k-1) | (nothing), innermost first
                for (long k = 0; k < hi - lo; ++k) {
                    const int32_t opt = g_.fresh_rule();
                    Alternative one = item;
                    if (inner >= 0) {
                        Symbol ref;
                        ref.rule = inner;
                        one.push_back(ref);
                    }
                    g_.rules_[opt] = {one, Alternative{}};
                    inner = opt;
                }
                if (inner >= 0) {
                    Symbol ref;
                    ref.rule = inner;
                    seq.push_back(ref);
                }
            }
        }
    };
};

// The grammar of one request and where its generation stands in it.
struct GrammarState {
    std::shared_ptr<const Grammar> grammar;
    std::string gbnf;
    std::vector<Grammar::Stack> stacks;
    std::string pending;        // bytes of an unfinished UTF-8 sequence carried over from the last token

    // Decodes `bytes` (after `carry`) into code points; the unfinished tail goes to `rest`.
    static void decode(const std::string & carry, const std::string & bytes, std::vector<uint32_t> & cps, std::string & rest) {
        const std::string all = carry + bytes;
        cps.clear();
        rest.clear();
        size_t i = 0;
        while (i < all.size()) {
            const unsigned char c = (unsigned char)all[i];
            const int extra = c >= 0xF0 ? 3 : c >= 0xE0 ? 2 : c >= 0xC0 ? 1 : 0;
            if (i + (size_t)extra + 1 > all.size()) {       // the sequence continues in the next token
                rest = all.substr(i);
                return;
            }
            uint32_t cp = extra == 3 ? c & 0x07 : extra == 2 ? c & 0x0F : extra == 1 ? c & 0x1F : c;
            for (int k = 1; k <= extra; ++k) cp = (cp << 6) | ((unsigned char)all[i + k] & 0x3F);
            cps.push_back(cp);
            i += (size_t)extra + 1;
        }
    }

    // Whether the token whose text is `piece` may come next (an end-of-generation token: only when the grammar is complete).
    bool allows(const std::string & piece, bool end_of_generation) const {
        if (end_of_generation) return pending.empty() && Grammar::complete(stacks);
        if (piece.empty()) return false;
        std::vector<uint32_t> cps;
        std::string rest;
        decode(pending, piece, cps, rest);
        if (!cps.empty() && !grammar->first_matches(stacks, cps[0])) return false;
        std::vector<Grammar::Stack> cur = stacks;
        for (uint32_t c : cps) {
            cur = grammar->accept(cur, c);
            if (cur.empty()) return false;
        }
        return rest.empty() || grammar->may_take_non_ascii(cur);
    }

    // Advances over the sampled token's text. False when the grammar rejects it (the state is then unchanged).
    bool advance(const std::string & piece, bool end_of_generation) {
        if (end_of_generation) return true;
        std::vector<uint32_t> cps;
        std::string rest;
        decode(pending, piece, cps, rest);
        std::vector<Grammar::Stack> cur = stacks;
        for (uint32_t c : cps) {
            cur = grammar->accept(cur, c);
            if (cur.empty()) return false;
        }
        stacks = std::move(cur);
        pending = rest;
        return true;
    }
};

} // namespace rb200
