// Checks the engine process's input half without a GPU: request lines from stdin are parsed and echoed field by field
// (or their error), and with --stop the STOP rule is run over a scripted input.
#include <cstdio>
#include <iostream>
#include <sstream>

#include "../../qwen3.8-flash-next-2x-p100_b200/csrc/serve_input.hpp"

int main(int argc, char** argv) {
    using namespace fnx_serve;
    if (argc > 1 && std::string(argv[1]) == "--stop") {
        // a STOP before the second request's line is for the first request only; one after the third's line for the third
        Input in;
        std::string line, out;
        long n = 0;
        for (const char* part : {"GEN 5 1,2\nSTOP\nPING\nGEN 3 4\n", "GEN 2 7\nSTOP\n"}) {
            std::istringstream is(part);
            in.run(is);
            in.eof = false;
            while (!in.lines.empty() && in.next(line, n)) {
                const bool stopped = n > 0 ? in.begin(n) : false;
                out += line.substr(0, line.find(' ')) + ":" + std::to_string(n) + ":" + (stopped ? "stopped" : "runs") + " ";
                if (n > 0) in.end();
            }
        }
        std::printf("%s\n", out.c_str());
        // a STOP that arrives while its request runs raises stop_now at once
        Input live;
        std::istringstream first("GEN 5 1\n");
        live.run(first);
        live.eof = false;
        live.next(line, n);
        live.begin(n);
        const bool before = live.stop_now.load();
        std::istringstream second("STOP\n");
        live.run(second);
        std::printf("%d %d\n", (int) before, (int) live.stop_now.load());
        // BSTOP <slot> is for that slot's latest BGEN line
        Input b;
        std::istringstream s1("BGEN 1 5 1,2\nBGEN 2 5 3\nBSTOP 1\n");
        b.run(s1);
        b.eof = false;
        long n1 = 0, n2 = 0, n3 = 0;
        b.next(line, n1);
        b.next(line, n2);
        const bool stop1 = b.bstopped(1, n1), stop2 = b.bstopped(2, n2);
        std::istringstream s2("BGEN 1 5 4\n");
        b.run(s2);
        b.next(line, n3);
        std::printf("%d %d %d %d\n", (int) stop1, (int) stop2, (int) b.bstopped(1, n3), (int) b.bstopped(1, n1));
        return 0;
    }
    std::string line;
    while (std::getline(std::cin, line)) {
        try {
            const bool batch = line.rfind("BGEN", 0) == 0;
            const Request r = parse_gen(line, 1000, batch, 4096);
            std::printf("OK slot=%d max_new=%d t=%g top_p=%g top_k=%d min_p=%g rep=%g freq=%g pres=%g last_n=%d seed=%s pen=%d bias=", r.slot, r.max_new, r.temperature,
                        r.top_p, r.top_k, r.min_p, r.pen_repeat, r.pen_freq, r.pen_present, r.pen_last_n, r.seed ? std::to_string(*r.seed).c_str() : "none",
                        (int) r.penalizes());
            for (auto& b : r.bias) std::printf("%d:%g;", b.first, b.second);
            std::printf(" ids=");
            for (int t : r.ids) std::printf("%d;", t);
            std::printf("\n");
        } catch (const std::exception& ex) {
            std::printf("ERR %s\n", ex.what());
        }
    }
    return 0;
}
