// The engine process's stdin and request lines (plain C++, no GPU): STOP acts the moment it arrives, every other line
// is queued; a request line (GEN <max_new> [key=value ...] <ids csv>) is parsed whole, each field named in its error.
// The counterpart of the reference's input half (engine/tools/sfnx_input.hpp:1-120, parse_gen engine/tools/sfnx.cpp:262-340).
#pragma once

#include <algorithm>
#include <atomic>
#include <cctype>
#include <cerrno>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <deque>
#include <istream>
#include <mutex>
#include <optional>
#include <sstream>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace fnx_serve {

constexpr int MAX_SLOTS = 8;

// STOP is for the latest request line that has come in and for no other: one sent before a request's line never acts on
// it, one sent after does however long the request waits in the queue.  BSTOP <slot> is for that slot's latest BGEN in the
// same way.
struct Input {
    std::mutex mu;
    std::condition_variable cv;
    std::deque<std::pair<std::string, long>> lines;   // the line and, for a request, its number (else 0)
    bool eof = false;
    long seq = 0;       // request lines so far
    long running = 0;   // the request the engine is on, 0: none
    long slot_seq[MAX_SLOTS] = {};   // the reader's own: the number of each slot's latest BGEN
    std::atomic<long> stop_upto{0}, bstop_upto[MAX_SLOTS];
    std::atomic<bool> stop_now{false};

    Input() {
        for (auto& b : bstop_upto) b = 0;
    }

    static bool is_request(const std::string& cmd) { return cmd == "GEN" || cmd == "BGEN"; }

    void run(std::istream& is) {
        std::string line;
        while (std::getline(is, line)) {
            if (!line.empty() && line.back() == '\r') line.pop_back();
            std::lock_guard<std::mutex> lk(mu);
            if (line == "STOP") {
                stop_upto = seq;
                if (running > 0 && running == seq) stop_now = true;
                continue;
            }
            int slot = -1;
            if (std::sscanf(line.c_str(), "BSTOP %d", &slot) == 1) {
                if (slot >= 0 && slot < MAX_SLOTS) bstop_upto[slot] = slot_seq[slot];
                continue;
            }
            const std::string cmd = line.substr(0, line.find(' '));
            long n = 0;
            if (is_request(cmd)) {
                n = ++seq;
                if (cmd == "BGEN" && std::sscanf(line.c_str() + 4, " %d", &slot) == 1 && slot >= 0 && slot < MAX_SLOTS) slot_seq[slot] = n;
            }
            lines.emplace_back(line, n);
            cv.notify_all();
        }
        std::lock_guard<std::mutex> lk(mu);
        eof = true;
        cv.notify_all();
    }

    // the next queued line: waits for one when `wait`, else answers only if one is there; false: none (see closed())
    bool next(std::string& line, long& n, bool wait = true) {
        std::unique_lock<std::mutex> lk(mu);
        if (wait) cv.wait(lk, [&] { return !lines.empty() || eof; });
        if (lines.empty()) return false;
        line = std::move(lines.front().first);
        n = lines.front().second;
        lines.pop_front();
        return true;
    }
    bool closed() {
        std::lock_guard<std::mutex> lk(mu);
        return eof && lines.empty();
    }

    // the engine takes up request n: true when a STOP for it is already in
    bool begin(long n) {
        std::lock_guard<std::mutex> lk(mu);
        running = n;
        stop_now = stop_upto.load() == n;
        return stop_now.load();
    }
    void end() {
        std::lock_guard<std::mutex> lk(mu);
        running = 0;
        stop_now = false;
    }
    // a BSTOP (or, for the request decoding there, a STOP) came for slot's request n
    bool bstopped(int slot, long n) const { return bstop_upto[slot].load() >= n || stop_upto.load() == n; }
};

struct Request {
    long seq = 0;
    int slot = -1;
    int max_new = 0;
    float temperature = 0.f, top_p = 1.f, min_p = 0.f;
    int top_k = 0;
    float pen_repeat = 1.f, pen_freq = 0.f, pen_present = 0.f;
    int pen_last_n = 64;
    std::optional<uint64_t> seed;
    std::vector<std::pair<int, float>> bias;   // logit_bias, sorted by token
    std::vector<int> ids;
    bool penalizes() const { return temperature > 0.f && pen_last_n > 0 && (pen_repeat != 1.f || pen_freq != 0.f || pen_present != 0.f); }
};

inline bool parse_whole(const std::string& v, long long& out) {
    if (v.empty()) return false;
    char* end = nullptr;
    errno = 0;
    out = std::strtoll(v.c_str(), &end, 10);
    return errno == 0 && end && *end == 0 && (std::isdigit((unsigned char) v[0]) || ((v[0] == '-' || v[0] == '+') && v.size() > 1));
}

inline bool parse_number(const std::string& v, double& out) {
    if (v.empty() || std::isspace((unsigned char) v[0])) return false;
    char* end = nullptr;
    errno = 0;
    out = std::strtod(v.c_str(), &end);
    return errno == 0 && end && *end == 0;
}

inline int field_int(const std::string& cmd, const std::string& key, const std::string& v) {
    long long x = 0;
    if (!parse_whole(v, x) || x < INT32_MIN || x > INT32_MAX) throw std::runtime_error(cmd + ": " + key + "=" + v + " is not a whole number");
    return (int) x;
}

inline float field_float(const std::string& cmd, const std::string& key, const std::string& v) {
    double x = 0;
    if (!parse_number(v, x) || !std::isfinite((float) x)) throw std::runtime_error(cmd + ": " + key + "=" + v + " is not a number");
    return (float) x;
}

// a comma-separated list's items, empty ones included ("1,,2" has three)
inline std::vector<std::string> split_commas(const std::string& s) {
    std::vector<std::string> out(1);
    for (char ch : s) {
        if (ch == ',') out.emplace_back();
        else out.back() += ch;
    }
    return out;
}

// the ranges of engine/src/session.cpp:140-151 (a greedy request's other values are not used and not checked)
inline void check_sampling(const Request& r, int pen_cap) {
    auto bad = [](const std::string& what) { throw std::runtime_error("sampling: " + what); };
    if (!std::isfinite(r.temperature) || r.temperature < 0.f) bad("temperature must be a finite number >= 0");
    if (r.temperature == 0.f) return;
    if (!(r.top_p > 0.f && r.top_p <= 1.f)) bad("top_p must be in (0, 1]");
    if (!(r.min_p >= 0.f && r.min_p <= 1.f)) bad("min_p must be in [0, 1]");
    if (r.top_k < 0) bad("top_k must be >= 0");
    if (!(std::isfinite(r.pen_repeat) && r.pen_repeat > 0.f)) bad("penalty_repeat must be a finite number > 0");
    if (!std::isfinite(r.pen_freq) || !std::isfinite(r.pen_present)) bad("penalty_freq and penalty_present must be finite");
    if (r.pen_last_n < 0) bad("penalty_last_n must be >= 0");
    if (r.penalizes() && r.pen_last_n > pen_cap) bad("penalty_last_n above " + std::to_string(pen_cap));
}

// GEN <max_new> [key=value ...] <ids csv>; BGEN <slot> <max_new> ...
inline Request parse_gen(const std::string& line, int vocab, bool batch, int pen_cap) {
    std::istringstream is(line);
    std::string cmd, word;
    Request r;
    is >> cmd;
    if (batch) {
        if (!(is >> word)) throw std::runtime_error(cmd + ": no slot");
        r.slot = field_int(cmd, "slot", word);
    }
    if (!(is >> word)) throw std::runtime_error(cmd + ": no max_new");
    r.max_new = field_int(cmd, "max_new", word);
    if (r.max_new < 1) throw std::runtime_error(cmd + ": max_new must be a number >= 1");
    std::string ids;
    while (is >> word) {
        const size_t eq = word.find('=');
        if (eq == std::string::npos) {
            ids = word;
            break;
        }
        const std::string k = word.substr(0, eq), v = word.substr(eq + 1);
        if (k == "temperature") r.temperature = field_float(cmd, k, v);
        else if (k == "top_p") r.top_p = field_float(cmd, k, v);
        else if (k == "top_k") r.top_k = field_int(cmd, k, v);
        else if (k == "min_p") r.min_p = field_float(cmd, k, v);
        else if (k == "penalty_repeat") r.pen_repeat = field_float(cmd, k, v);
        else if (k == "penalty_freq") r.pen_freq = field_float(cmd, k, v);
        else if (k == "penalty_present") r.pen_present = field_float(cmd, k, v);
        else if (k == "penalty_last_n") r.pen_last_n = field_int(cmd, k, v);
        else if (k == "seed") {   // 0 to 2^64 - 1
            if (v.empty() || v.size() > 20 || v.find_first_not_of("0123456789") != std::string::npos || (v.size() == 20 && v > "18446744073709551615"))
                throw std::runtime_error(cmd + ": seed=" + v + " is not a whole number from 0 to 2^64-1");
            r.seed = std::stoull(v);
        } else if (k == "logit_bias") {
            for (const std::string& e : split_commas(v)) {
                const size_t c = e.find(':');
                long long id = -1;
                if (c == std::string::npos || !parse_whole(e.substr(0, c), id) || id < 0 || id >= vocab)
                    throw std::runtime_error(cmd + ": logit_bias entry '" + e.substr(0, 40) + "' is not <token id>:<bias> within the vocabulary");
                const float b = field_float(cmd, "logit_bias", e.substr(c + 1));
                if (b < -100.f || b > 100.f) throw std::runtime_error(cmd + ": logit_bias " + e.substr(0, 40) + ": a bias is from -100 to 100");
                r.bias.emplace_back((int) id, b);
            }
            std::sort(r.bias.begin(), r.bias.end());
            for (size_t i = 1; i < r.bias.size(); ++i)
                if (r.bias[i].first == r.bias[i - 1].first) throw std::runtime_error(cmd + ": logit_bias names token " + std::to_string(r.bias[i].first) + " twice");
        } else if (k == "keep" || k == "ckpt" || k == "pin" || k == "pcie_frac" || k == "spec_min_p" || k == "pipe" || k == "aux_cpus" || k == "cvec") {
            // cache hints and the front end's per-request engine tuning: nothing in this engine to set, the request goes on
        } else {
            throw std::runtime_error(cmd + ": unknown key " + k);
        }
    }
    if (is >> word) throw std::runtime_error(cmd + ": text after the token ids");
    if (ids.empty()) throw std::runtime_error(cmd + ": no token ids");
    try {
        check_sampling(r, pen_cap);
    } catch (const std::runtime_error& ex) {
        throw std::runtime_error(cmd + ": " + ex.what());
    }
    for (const std::string& t : split_commas(ids)) {
        long long v = 0;
        if (!parse_whole(t, v)) throw std::runtime_error(cmd + ": token id '" + t + "' is not a whole number");
        if (v < 0 || v >= vocab) throw std::runtime_error(cmd + ": token id " + t + " outside the vocabulary");
        r.ids.push_back((int) v);
    }
    return r;
}

}  // namespace fnx_serve
