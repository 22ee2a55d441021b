// The engine process for a front end that speaks the reference's line protocol (engine/tools/sfnx.cpp:1-19): token ids
// in, token ids out, on stdin / stdout.  The server tokenizes, applies the chat template and matches stop strings.
//
//   fnx_serve --serve --native MODEL.gguf [--max-context N] [--spec K] [--lookup K] [--eos ID,ID] [--batch SLOTS]
//             [--conversation-cache-mib M]
//
// After loading: INFO engine=fnx_b200 ... and READY <max context> stop.  One request at a time:
//   GEN <max_new> [key=value ...] <ids csv>
// answered with PP <done> <total> per prompt chunk, RESUME <reused>, T <id> per token (speculative: the draft layer's
// chain and n-gram lookups, verified a window at a time), DONE <generated> <prompt_tokens> <prompt_ms> <decode_ms> <finish>
// <drafts_accepted> <drafts_offered> <reused>, or ERR <why>.  STOP at any time ends the latest request (finish "cancel").
// QUIT (or the end of the input) ends the process.  Keys: temperature top_p top_k min_p seed (sampling: the engine's
// speculative-sampling rule over each row's 64 best tokens); penalty_repeat penalty_freq penalty_present penalty_last_n (sampled
// requests) and logit_bias=<id>:<bias>,... (greedy ones too) change each window row's logits before the rule looks at them.
// A prompt that extends what the engine already holds reads only its new tokens (RESUME counts the reused ones).  With
// --conversation-cache-mib M a conversation that another one displaces is parked in host memory (the engine's sequence state:
// K/V rows, DeltaNet states, context) and comes back when a later prompt goes on from it; the least recently used go first.
// With --batch (INFO batch_slots=N): BGEN <slot> <max_new> <ids csv> reads a prompt into a free slot (each slot one of the
// engine's sequences) between the decoding slots' windows and answers its first token as T + DONE, then BADM <slot> 1 if it
// goes on (0 if not); the decoding slots share windows (a row each and their draft-layer drafts: the engine's batched lanes)
// and stream BT <slot> <id> ... BDONE <slot> <produced> <finish> <ms> <drafts_accepted> <drafts_offered> <rounds>.  BSTOP <slot>
// ends a decoding slot, or its prompt read at the next chunk.  Batched slots decode greedily; sampled requests run as GEN.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <random>
#include <string>
#include <thread>
#include <vector>

#include "../../include/fnx_b200.h"
#include "serve_input.hpp"

namespace {

using fnx_serve::Input;
using fnx_serve::Request;

void say(const std::string& line) {
    std::fwrite(line.data(), 1, line.size(), stdout);
    std::fputc('\n', stdout);
    std::fflush(stdout);
}

struct Args {
    std::string gguf;
    int max_ctx = 32768, K = 4, lookup = 15, prompt_chunk = 8192, batch = 1;
    long cache_mib = 0;   // parked conversations in host memory (0: none)
    std::vector<int> eos;
};

Args parse_args(int argc, char** argv) {
    Args a;
    bool serve = false;
    for (int i = 1; i < argc; ++i) {
        const std::string k = argv[i];
        auto val = [&]() -> std::string {
            if (i + 1 >= argc) throw std::runtime_error(k + " needs a value");
            return argv[++i];
        };
        if (k == "--serve") serve = true;
        else if (k == "--native") a.gguf = val();
        else if (k == "--max-context") a.max_ctx = std::stoi(val());
        else if (k == "--spec") a.K = std::stoi(val());
        else if (k == "--lookup") a.lookup = std::stoi(val());
        else if (k == "--prompt-chunk") a.prompt_chunk = std::stoi(val());
        else if (k == "--eos") {
            for (const std::string& t : fnx_serve::split_commas(val())) a.eos.push_back(fnx_serve::field_int("--eos", "id", t));
        }
        // the reference's draft-layer files and card layout: this engine's file holds the draft layer, one GPU holds the model
        else if (k == "--conversation-cache-mib") a.cache_mib = std::stol(val());
        else if (k == "--mtp" || k == "--draft-vocab" || k == "--layer-split") val();
        else if (k == "--batch") a.batch = std::stoi(val());
        else throw std::runtime_error("unknown argument " + k);
    }
    if (!serve) throw std::runtime_error("fnx_serve runs as --serve");
    if (a.gguf.empty()) throw std::runtime_error("--native is required");
    if (a.K < 0 || a.K > FNX_MAX_ROWS - 1) throw std::runtime_error("--spec must be 0.." + std::to_string(FNX_MAX_ROWS - 1));
    if (a.lookup < 0 || a.lookup > FNX_MAX_ROWS - 1) throw std::runtime_error("--lookup must be 0.." + std::to_string(FNX_MAX_ROWS - 1));
    if (a.max_ctx < 16) throw std::runtime_error("--max-context must be at least 16");
    if (a.prompt_chunk < 1) throw std::runtime_error("--prompt-chunk must be at least 1");
    if (a.cache_mib < 0) throw std::runtime_error("--conversation-cache-mib must be >= 0");
    if (a.batch < 1 || a.batch > fnx_serve::MAX_SLOTS) throw std::runtime_error("--batch must be 1.." + std::to_string(fnx_serve::MAX_SLOTS));
    return a;
}

double ms_since(std::chrono::steady_clock::time_point t) {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t).count();
}

void ok(int rc, const char* what) {
    if (rc != FNX_OK) throw std::runtime_error(std::string(what) + ": " + fnx_last_error());
}

struct Server {
    const Args& a;
    fnx_engine* e;
    fnx_model_config c;
    Input& in;
    std::vector<int> history;   // the tokens sequence 0 holds
    bool sampling = false;      // the acceptance rule the engine is set to
    bool rules = false;         // the engine applies a request's penalties or logit_bias
    struct Parked {
        std::vector<int> tokens;       // the conversation's kept tokens
        std::vector<uint8_t> state;    // fnx_engine_save_state's image, K/V rows included
        long used = 0;
    };
    std::vector<Parked> parked;
    size_t parked_bytes = 0;
    long clock = 0;
    struct Slot {
        bool decoding = false;
        long seq = 0;               // its request's number
        int max_new = 0, produced = 0, rounds = 0;
        int x = 0;                  // the next window's first row: the last token it emitted
        std::vector<int> drafts;
        long accepted = 0, offered = 0;
        std::chrono::steady_clock::time_point t0;
    };
    std::vector<Slot> slots;
    bool dirty = false;         // a request failed half way: the engine's sequence is not `history`

    bool is_eos(int t) const {
        for (int x : a.eos)
            if (x == t) return true;
        return false;
    }

    void set_rule(const Request& r) {
        if (r.temperature == 0.f) {
            if (sampling) ok(fnx_engine_set_sampling(e, nullptr, 0), "set_sampling");
            sampling = false;
            return;
        }
        // every sampled request sets the rule anew: the engine's uniforms are addressed (seed, sequence, window), and the window
        // count starts over with the rule, so a seeded request draws the same tokens whatever ran before it
        const fnx_sampling s{r.temperature, r.top_p, r.min_p, r.top_k};
        const uint64_t seed = r.seed ? *r.seed : ((uint64_t) std::random_device{}() << 32) ^ std::random_device{}();
        ok(fnx_engine_set_sampling(e, &s, seed), "set_sampling");
        sampling = true;
    }

    // the request's penalties (sampled requests only, as the reference's penalizes()) and logit_bias (greedy ones too)
    void set_logit_rules(const Request& r) {
        if (!r.penalizes() && r.bias.empty()) {
            if (rules) ok(fnx_engine_set_logit_rules(e, nullptr), "set_logit_rules");
            rules = false;
            return;
        }
        std::vector<int> bt;
        std::vector<float> bv;
        for (const auto& b : r.bias) bt.push_back(b.first), bv.push_back(b.second);
        fnx_logit_rules lr{};
        lr.repeat = r.pen_repeat, lr.freq = r.pen_freq, lr.present = r.pen_present;
        lr.last_n = r.penalizes() ? r.pen_last_n : 0;
        lr.bias_tok = bt.data(), lr.bias_val = bv.data(), lr.bias_n = (int) bt.size();
        ok(fnx_engine_set_logit_rules(e, &lr), "set_logit_rules");
        rules = true;
    }

    // the live conversation of sequence 0 to host memory, if the cache has (or can make) room for it
    void park_live() {
        const size_t budget = (size_t) a.cache_mib << 20;
        if (dirty || history.empty() || budget == 0) return;
        const size_t need = fnx_engine_state_bytes(e, 0, 1);
        if (need == 0 || need > budget) return;
        while (parked_bytes + need > budget && !parked.empty()) {   // the least recently used go first
            size_t lru = 0;
            for (size_t i = 1; i < parked.size(); ++i)
                if (parked[i].used < parked[lru].used) lru = i;
            parked_bytes -= parked[lru].state.size();
            parked.erase(parked.begin() + (long) lru);
        }
        Parked p;
        p.tokens = history;
        p.state.resize(need);
        p.used = ++clock;
        ok(fnx_engine_save_state(e, 0, 1, p.state.data(), need), "save_state");
        parked_bytes += need;
        parked.push_back(std::move(p));
    }

    // the longest parked conversation that the prompt (all but its last token) goes on from: back into sequence 0
    size_t unpark_for(const std::vector<int>& ids) {
        int best = -1;
        for (size_t i = 0; i < parked.size(); ++i) {
            const std::vector<int>& t = parked[i].tokens;
            if (t.size() <= ids.size() - 1 && std::equal(t.begin(), t.end(), ids.begin()) && (best < 0 || t.size() > parked[(size_t) best].tokens.size())) best = (int) i;
        }
        if (best < 0) return 0;
        Parked& p = parked[(size_t) best];
        ok(fnx_engine_load_state(e, 0, p.state.data(), p.state.size()), "load_state");
        history = p.tokens;
        parked_bytes -= p.state.size();
        parked.erase(parked.begin() + best);
        return history.size();
    }

    void solo(const Request& r) {
        const bool stopped = in.begin(r.seq);
        struct End {
            Input& in;
            ~End() { in.end(); }
        } end{in};
        const int n = (int) r.ids.size();
        // what the engine holds of this prompt: all of its history, when the prompt goes on from it (its last token is read by the first window)
        size_t reused = 0;
        if (!dirty && history.size() <= (size_t) n - 1 && std::equal(history.begin(), history.end(), r.ids.begin())) reused = history.size();
        else {
            park_live();   // another conversation takes the sequence: this one waits in host memory
            history.clear();
            if (dirty) ok(fnx_engine_reset(e, 0), "reset");   // (a request that failed half way may have left a window open)
            reused = unpark_for(r.ids);
            if (reused == 0) ok(fnx_engine_reset(e, 0), "reset");
        }
        dirty = true;
        set_rule(r);
        set_logit_rules(r);
        const auto t0 = std::chrono::steady_clock::now();
        bool cancelled = stopped;
        for (int at = (int) reused; at < n - 1 && !cancelled;) {
            const int m = std::min(a.prompt_chunk, n - 1 - at);
            ok(fnx_engine_prompt(e, 0, r.ids.data() + at, m), "prompt");
            history.insert(history.end(), r.ids.begin() + at, r.ids.begin() + at + m);
            at += m;
            say("PP " + std::to_string(at) + " " + std::to_string(n - 1));
            cancelled = in.stop_now.load();
        }
        const double prompt_ms = ms_since(t0);
        say("RESUME " + std::to_string(reused));
        int generated = 0;
        long accepted = 0, offered = 0;
        const char* finish = "length";
        const auto t1 = std::chrono::steady_clock::now();
        if (cancelled) finish = "cancel";
        else {
            int x = r.ids.back();
            std::vector<int> drafts;
            int result[1 + 2 * FNX_MAX_ROWS];
            for (;;) {
                if (in.stop_now.load()) {
                    finish = "cancel";
                    break;
                }
                const int room = c.max_ctx - fnx_engine_pos(e, 0) - 1;
                if (room < 0) break;
                if ((int) drafts.size() > room) drafts.resize((size_t) room);
                if ((int) drafts.size() > c.max_rows - 1) drafts.resize((size_t) c.max_rows - 1);
                std::vector<int> rows{x};
                rows.insert(rows.end(), drafts.begin(), drafts.end());
                ok(fnx_engine_verify(e, 0, rows.data(), nullptr, (int) rows.size(), result), "verify");
                const int n_acc = result[0];
                const int* path = result + 1;
                const int* out = result + 1 + FNX_MAX_ROWS;
                // emit the accepted drafts' successors in order until a stop: the window keeps the rows before the last emitted
                int used = 0;
                bool done = false;
                for (int j = 0; j < n_acc && !done; ++j) {
                    say("T " + std::to_string(out[j]));
                    ++used;
                    ++generated;
                    if (is_eos(out[j])) finish = "stop", done = true;
                    else if (generated >= r.max_new) finish = "length", done = true;
                }
                ok(fnx_engine_commit(e, 0, path, used), "commit");
                history.insert(history.end(), rows.begin(), rows.begin() + used);
                offered += (long) drafts.size();
                accepted += used - 1;
                x = out[used - 1];
                // the draft layer reads the kept rows either way: its cells stay current for a later request that goes on from here
                drafts.clear();
                std::vector<int> chain((size_t) std::max(a.K, 1));
                if (a.K > 0) ok(fnx_engine_draft(e, 0, done ? 1 : a.K, chain.data()), "draft");
                if (done) break;
                if (a.K > 0) {
                    // n-gram lookup first (the tokens after the latest earlier place of the context's end, if they start with the
                    // draft layer's first token); else the draft layer's chain
                    int lk[FNX_MAX_ROWS], n_lk = 0;
                    if (a.lookup > 0) ok(fnx_engine_lookup(e, 0, a.lookup, chain[0], x, lk, &n_lk), "lookup");
                    if (n_lk > 0) drafts.assign(lk, lk + n_lk);
                    else drafts = chain;
                }
            }
        }
        char buf[256];
        std::snprintf(buf, sizeof buf, "DONE %d %d %.1f %.1f %s %ld %ld %zu", generated, (int) std::min(history.size(), (size_t) n), prompt_ms, ms_since(t1), finish,
                      accepted, offered, reused);
        say(buf);
        dirty = false;
    }

    bool any_decoding() const {
        for (const Slot& sl : slots)
            if (sl.decoding) return true;
        return false;
    }

    // batched slots decode greedily, without logit rules: whatever a solo request set goes
    void plain_rule() {
        if (sampling) ok(fnx_engine_set_sampling(e, nullptr, 0), "set_sampling");
        if (rules) ok(fnx_engine_set_logit_rules(e, nullptr), "set_logit_rules");
        sampling = rules = false;
    }

    void finish_slot(int i, const char* finish) {
        Slot& sl = slots[(size_t) i];
        char buf[160];
        std::snprintf(buf, sizeof buf, "BDONE %d %d %s %.1f %ld %ld %d", i, sl.produced, finish, ms_since(sl.t0), sl.accepted, sl.offered, sl.rounds);
        say(buf);
        sl.decoding = false;
    }

    // drafts a lane may carry: the chain, as far as the window's rows go round the decoding slots
    int lane_drafts(int lanes) const { return std::max(0, std::min({a.K, FNX_LANE_ROWS - 1, c.max_rows / std::max(lanes, 1) - 1})); }

    // BGEN: the prompt into the slot's sequence, its first token through a window of that sequence alone
    void admit(const Request& r) {
        const int i = r.slot;
        if (i < 0 || i >= (int) slots.size() || slots[(size_t) i].decoding)
            throw std::runtime_error("BGEN: no such free slot " + std::to_string(i) + " (--batch " + std::to_string(slots.size()) + ")");
        if (r.temperature != 0.f || !r.bias.empty())
            throw std::runtime_error("BGEN: batched slots decode greedily (sampling, penalties and logit_bias run as GEN)");
        plain_rule();
        Slot& sl = slots[(size_t) i];
        sl = Slot{};
        sl.seq = r.seq;
        if (i == 0) history.clear(), dirty = true;   // sequence 0 is also the solo requests'
        ok(fnx_engine_reset(e, i), "reset");
        const int n = (int) r.ids.size();
        const auto t0 = std::chrono::steady_clock::now();
        auto done_line = [&](int generated, int read, double decode_ms, const char* finish) {
            char buf[256];
            std::snprintf(buf, sizeof buf, "DONE %d %d %.1f %.1f %s 0 0 0", generated, read, ms_since(t0) - decode_ms, decode_ms, finish);
            say(buf);
        };
        int at = 0;
        bool cancelled = in.bstopped(i, r.seq);
        while (at < n - 1 && !cancelled) {
            const int m = std::min(a.prompt_chunk, n - 1 - at);
            ok(fnx_engine_prompt(e, i, r.ids.data() + at, m), "prompt");
            at += m;
            say("PP " + std::to_string(at) + " " + std::to_string(n - 1));
            cancelled = in.bstopped(i, r.seq);
        }
        say("RESUME 0");
        if (cancelled) {
            done_line(0, at, 0.0, "cancel");
            say("BADM " + std::to_string(i) + " 0");
            return;
        }
        const auto t1 = std::chrono::steady_clock::now();
        int result[1 + 2 * FNX_MAX_ROWS];
        const int x = r.ids.back();
        ok(fnx_engine_verify(e, i, &x, nullptr, 1, result), "verify");
        const int tok = result[1 + FNX_MAX_ROWS], keep = 0;
        ok(fnx_engine_commit(e, i, &keep, 1), "commit");
        say("T " + std::to_string(tok));
        const bool more = !is_eos(tok) && r.max_new > 1;
        // its first drafts (and the draft layer's cells for the kept row)
        std::vector<int> chain((size_t) std::max(a.K, 1));
        if (a.K > 0) ok(fnx_engine_draft(e, i, more ? a.K : 1, chain.data()), "draft");
        done_line(1, n, ms_since(t1), is_eos(tok) ? "stop" : "length");
        say("BADM " + std::to_string(i) + (more ? " 1" : " 0"));
        if (!more) return;
        sl.decoding = true;
        sl.max_new = r.max_new;
        sl.produced = 1;
        sl.x = tok;
        sl.drafts = a.K > 0 ? chain : std::vector<int>{};
        sl.t0 = std::chrono::steady_clock::now();
    }

    // one window of every decoding slot: a row each and their drafts, accepted greedily per lane
    void decode_step() {
        std::vector<int> lanes;
        for (int i = 0; i < (int) slots.size(); ++i) {
            Slot& sl = slots[(size_t) i];
            if (!sl.decoding) continue;
            if (in.bstopped(i, sl.seq)) finish_slot(i, "cancel");
            else if (fnx_engine_pos(e, i) + 1 > c.max_ctx) finish_slot(i, "length");
            else lanes.push_back(i);
        }
        if (lanes.empty()) return;
        plain_rule();
        const int nl = (int) lanes.size(), kd = lane_drafts(nl);
        std::vector<int> rows((size_t) nl), tok, results((size_t) nl * (1 + 2 * FNX_MAX_ROWS)), keep((size_t) nl);
        for (int j = 0; j < nl; ++j) {
            Slot& sl = slots[(size_t) lanes[(size_t) j]];
            const int room = c.max_ctx - fnx_engine_pos(e, lanes[(size_t) j]) - 1;
            if ((int) sl.drafts.size() > std::min(kd, room)) sl.drafts.resize((size_t) std::max(0, std::min(kd, room)));
            rows[(size_t) j] = 1 + (int) sl.drafts.size();
            tok.push_back(sl.x);
            tok.insert(tok.end(), sl.drafts.begin(), sl.drafts.end());
        }
        ok(fnx_engine_verify_lanes_rows(e, nl, lanes.data(), rows.data(), tok.data(), results.data()), "verify_lanes");
        std::vector<bool> done((size_t) nl, false);
        std::vector<const char*> why((size_t) nl, "length");
        for (int j = 0; j < nl; ++j) {
            Slot& sl = slots[(size_t) lanes[(size_t) j]];
            const int* res = results.data() + (size_t) j * (1 + 2 * FNX_MAX_ROWS);
            const int n_acc = res[0];
            const int* out = res + 1 + FNX_MAX_ROWS;
            int used = 0;
            for (int t = 0; t < n_acc && !done[(size_t) j]; ++t) {
                say("BT " + std::to_string(lanes[(size_t) j]) + " " + std::to_string(out[t]));
                ++used;
                ++sl.produced;
                if (is_eos(out[t])) why[(size_t) j] = "stop", done[(size_t) j] = true;
                else if (sl.produced >= sl.max_new) why[(size_t) j] = "length", done[(size_t) j] = true;
            }
            keep[(size_t) j] = used;
            sl.offered += (long) sl.drafts.size();
            sl.accepted += used - 1;
            ++sl.rounds;
            sl.x = out[used - 1];
        }
        ok(fnx_engine_commit_lanes(e, nl, lanes.data(), keep.data()), "commit_lanes");
        // the draft layer reads every lane's kept rows; the lanes that go on take its chain as their next drafts
        const int kn = std::max(1, std::min(a.K, FNX_LANE_ROWS - 1));
        std::vector<int> drafts((size_t) nl * kn);
        if (a.K > 0) ok(fnx_engine_draft_lanes(e, nl, lanes.data(), kn, drafts.data()), "draft_lanes");
        for (int j = 0; j < nl; ++j) {
            Slot& sl = slots[(size_t) lanes[(size_t) j]];
            if (done[(size_t) j]) finish_slot(lanes[(size_t) j], why[(size_t) j]);
            else if (a.K > 0) sl.drafts.assign(drafts.begin() + (size_t) j * kn, drafts.begin() + (size_t) (j + 1) * kn);
        }
    }

    void run() {
        std::string line;
        long seq = 0;
        for (;;) {
            // requests first; the decoding slots' window when none is waiting
            if (!in.next(line, seq, !any_decoding())) {
                if (!any_decoding() && in.closed()) return;
                try {
                    decode_step();
                } catch (const std::exception& ex) {   // the window failed: its slots end, the process carries on
                    say(std::string("ERR ") + ex.what());
                    for (int i = 0; i < (int) slots.size(); ++i)
                        if (slots[(size_t) i].decoding) finish_slot(i, "cancel");
                }
                continue;
            }
            if (line.empty()) continue;
            const std::string cmd = line.substr(0, line.find(' '));
            if (cmd == "QUIT") return;
            if (cmd != "GEN" && cmd != "BGEN") {
                say("ERR " + cmd + ": not supported by fnx_serve");
                continue;
            }
            const bool batch = cmd == "BGEN";
            if (batch && slots.size() < 2) {
                say("ERR BGEN: fnx_serve runs without --batch");
                continue;
            }
            try {
                Request r = fnx_serve::parse_gen(line, c.vocab, batch, FNX_PENALTY_CAP);
                if ((long) r.ids.size() + r.max_new + 8 > c.max_ctx) throw std::runtime_error(cmd + ": prompt + max_new exceed the context");
                r.seq = seq;
                if (batch) admit(r);
                else if (slots[0].decoding) throw std::runtime_error("GEN: slot 0 is decoding (a solo request runs on its sequence)");
                else solo(r);
            } catch (const std::exception& ex) {
                say(std::string("ERR ") + ex.what());
            }
        }
    }
};

}  // namespace

int main(int argc, char** argv) {
    Args a;
    try {
        a = parse_args(argc, argv);
    } catch (const std::exception& ex) {
        std::fprintf(stderr, "fnx_serve: %s\n", ex.what());
        return 2;
    }
    const auto t_load = std::chrono::steady_clock::now();
    fnx_gguf* g = nullptr;
    fnx_engine* e = nullptr;
    fnx_model_config c{};
    int converted = 0;
    try {
        ok(fnx_gguf_open(a.gguf.c_str(), &g), "open");
        c.max_ctx = a.max_ctx;
        c.max_rows = std::max({8, std::max(a.K, a.lookup) + 1, std::min((int) FNX_MAX_ROWS, a.batch * (1 + std::min(a.K, FNX_LANE_ROWS - 1)))});
        c.n_seq = a.batch;
        c.ep_rank = 0;
        c.ep_size = 1;
        ok(fnx_gguf_model_config(g, &c), "model file");
        ok(fnx_engine_create(&c, &e), "engine");
        ok(fnx_engine_load_gguf(e, g, &converted), "load");
        double eos = 0;   // the tokenizer's end-of-sequence token, when the file names one and the command line none
        if (a.eos.empty() && fnx_gguf_num(g, "tokenizer.ggml.eos_token_id", &eos)) a.eos.push_back((int) eos);
        fnx_gguf_close(g);
        g = nullptr;
    } catch (const std::exception& ex) {
        say(std::string("ERR ") + ex.what());
        return 1;
    }
    std::fprintf(stderr, "fnx_serve: loaded in %.1f s (%d tensors quantised to IQ3_S on the way), %.2f GiB on the GPU, context %d, chain %d, lookup %d\n",
                 ms_since(t_load) / 1e3, converted, fnx_engine_device_bytes(e) / 1073741824.0, a.max_ctx, a.K, a.lookup);
    say("INFO engine=fnx_b200 version=" + std::to_string(fnx_version()) + " spec=" + std::to_string(a.K) + " conversation_cache_mib=" + std::to_string(a.cache_mib) + " logit_bias=1" +
        (a.batch > 1 ? " batch_slots=" + std::to_string(a.batch) : ""));
    say("READY " + std::to_string(a.max_ctx) + " stop");
    Input in;
    std::thread reader([&] { in.run(std::cin); });
    reader.detach();
    Server srv{a, e, c, in};
    srv.slots.resize((size_t) a.batch);
    try {
        srv.run();
    } catch (const std::exception& ex) {
        say(std::string("ERR ") + ex.what());
        std::fflush(stdout);
        std::_Exit(1);
    }
    std::fflush(stdout);
    std::_Exit(0);   // the reader may still sit in getline
}
