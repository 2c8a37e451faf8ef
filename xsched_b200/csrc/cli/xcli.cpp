// xcli — command-line client of the scheduling server's control interface.
//
//   xcli [-a ADDR] [-p PORT] list                         one table of every XQueue the server knows
//   xcli ... top [-f FPS]                                 the same table, redrawn until interrupted
//   xcli ... config -x HANDLE [-l LEVEL] [-t THRESHOLD] [-b BATCH]
//   xcli ... policy -q | policy -s -n NAME                query / hot-swap the server's policy
//   xcli ... hint -x HANDLE -p PRIORITY | -u UTILIZATION  |  hint --pid PID -u UTILIZATION  |  hint -t TIMESLICE_US
//
// Sub-commands and options are those of the reference's xcli (service/cli/src/main.cpp:11-110); the tables are
// plain text (the reference draws them with a terminal UI library that is not available here).
#include <algorithm>
#include <chrono>
#include <csignal>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <thread>
#include <vector>

#include "server/http.h"
#include "xsched/protocol/def.h"
#include "xsched/protocol/names.h"
#include "xsched/sched/wire.h"
#include "xsched/xsched.h"

using xsched::service::HttpCall;

namespace {

struct Options {
    std::string addr = "127.0.0.1";
    int port = XSCHED_SERVER_DEFAULT_PORT;
};

int Usage() {
    std::fprintf(stderr,
                 "usage: xcli [-a ADDR] [-p PORT] <command>\n"
                 "  list                                   list the XQueues known to the server\n"
                 "  top [-f FPS]                           keep listing (default 1 per second)\n"
                 "  config -x HANDLE [-l 1|2|3] [-t THRESHOLD] [-b BATCH_SIZE]\n"
                 "  policy -q | policy -s -n NAME          query or set the scheduling policy\n"
                 "  hint -x HANDLE -p PRIORITY | -x HANDLE -u UTIL | --pid PID -u UTIL | -t TIMESLICE_US\n");
    return 1;
}

// Splits the top-level members of the array found after "key": [ ... ] into object texts.
std::vector<std::string> ObjectsOf(const std::string &json, const std::string &key) {
    std::vector<std::string> out;
    size_t p = json.find("\"" + key + "\"");
    if (p == std::string::npos) return out;
    p = json.find('[', p);
    if (p == std::string::npos) return out;
    int depth = 0;
    size_t begin = 0;
    bool in_str = false;
    for (size_t i = p + 1; i < json.size(); ++i) {
        const char c = json[i];
        if (in_str) { if (c == '\\') ++i; else if (c == '"') in_str = false; continue; }
        if (c == '"') in_str = true;
        else if (c == '{') { if (depth++ == 0) begin = i; }
        else if (c == '}') { if (--depth == 0) out.push_back(json.substr(begin, i - begin + 1)); }
        else if (c == ']' && depth == 0) break;
    }
    return out;
}

int Fetch(const Options &o, const std::string &method, const std::string &target, const std::string &body, std::string *out) {
    const int status = HttpCall(o.addr, (uint16_t)o.port, method, target, body, out);
    if (status == 0) std::fprintf(stderr, "xcli: cannot reach the server at %s:%d\n", o.addr.c_str(), o.port);
    return status;
}

int List(const Options &o) {
    std::string body;
    const int status = Fetch(o, "GET", "/xqueues", "", &body);
    if (status != 200) { if (status) std::fprintf(stderr, "xcli: server answered %d\n", status); return 1; }
    std::map<std::string, std::string> cmd_of;
    for (const std::string &p : ObjectsOf(body, "processes")) {
        std::map<std::string, std::string> m;
        if (xsched::service::ParseFlatJson(p, &m)) cmd_of[m["pid"]] = m["cmdline"];
    }
    std::vector<std::map<std::string, std::string>> rows;
    for (const std::string &q : ObjectsOf(body, "xqueues")) {
        std::map<std::string, std::string> m;
        if (xsched::service::ParseFlatJson(q, &m)) rows.push_back(m);
    }
    std::sort(rows.begin(), rows.end(), [](auto &a, auto &b) { return std::atoll(a["pid"].c_str()) < std::atoll(b["pid"].c_str()); });
    std::printf("%8s  %-18s  %-18s  %-4s  %-5s  %2s  %9s  %5s  %s\n", "PID", "DEV", "XQUEUE", "STAT", "SCHED", "LV", "THRESHOLD", "BATCH", "CMD");
    for (auto &m : rows) {
        char dev[32], xq[32];
        std::snprintf(dev, sizeof(dev), "0x%llx", std::strtoull(m["device"].c_str(), nullptr, 10));
        std::snprintf(xq, sizeof(xq), "0x%llx", std::strtoull(m["handle"].c_str(), nullptr, 10));
        std::printf("%8s  %-18s  %-18s  %-4s  %-5s  %2s  %9s  %5s  %s\n", m["pid"].c_str(), dev, xq, m["ready"] == "true" ? "RDY" : "BLK",
                    m["suspended"] == "true" ? "SUS" : "RUN", m["level"].c_str(), m["threshold"].c_str(), m["batch_size"].c_str(), cmd_of[m["pid"]].c_str());
    }
    std::printf("%zu XQueue(s)\n", rows.size());
    return 0;
}

volatile std::sig_atomic_t g_stop = 0;

int Top(const Options &o, double fps) {
    std::signal(SIGINT, [](int) { g_stop = 1; });
    while (!g_stop) {
        std::printf("\033[2J\033[H");
        if (List(o) != 0) return 1;
        std::fflush(stdout);
        std::this_thread::sleep_for(std::chrono::milliseconds((int)(1000.0 / fps)));
    }
    return 0;
}

int Report(int status, const std::string &body) {
    std::printf("%s\n", body.empty() ? (status == 200 ? "{}" : "") : body.c_str());
    return status == 200 ? 0 : 1;
}

} // namespace

int main(int argc, char **argv) {
    Options o;
    int i = 1;
    for (; i + 1 < argc && argv[i][0] == '-'; i += 2) {
        if (!std::strcmp(argv[i], "-a") || !std::strcmp(argv[i], "--addr")) o.addr = argv[i + 1];
        else if (!std::strcmp(argv[i], "-p") || !std::strcmp(argv[i], "--port")) o.port = std::atoi(argv[i + 1]);
        else return Usage();
    }
    if (i >= argc) return Usage();
    const std::string cmd = argv[i++];
    std::map<std::string, std::string> opt;
    for (; i < argc; ++i) {
        const std::string k = argv[i];
        if (k == "-q" || k == "--query" || k == "-s" || k == "--set") { opt[k.substr(0, 2) == "--" ? k.substr(2, 1).insert(0, "-") : k] = "1"; continue; }
        if (i + 1 >= argc) return Usage();
        opt[k] = argv[++i];
    }
    auto get = [&](const char *a, const char *b) -> std::string { auto it = opt.find(a); if (it != opt.end()) return it->second; it = opt.find(b); return it == opt.end() ? "" : it->second; };

    if (cmd == "list") return List(o);
    if (cmd == "top") { const std::string f = get("-f", "--frequency"); return Top(o, f.empty() ? 1.0 : std::max(0.1, std::atof(f.c_str()))); }
    if (cmd == "config") {
        const std::string x = get("-x", "--xqueue");
        if (x.empty()) return Usage();
        char target[256];
        std::string query;
        const std::string l = get("-l", "--level"), t = get("-t", "--threshold"), b = get("-b", "--batch-size");
        if (!l.empty()) query += "level=" + l + "&";
        if (!t.empty()) query += "threshold=" + t + "&";
        if (!b.empty()) query += "batch_size=" + b + "&";
        std::snprintf(target, sizeof(target), "/config/%llx%s%s", std::strtoull(x.c_str(), nullptr, 0), query.empty() ? "" : "?", query.c_str());
        std::string body;
        return Report(Fetch(o, "POST", target, "", &body), body);
    }
    if (cmd == "policy") {
        std::string body;
        if (opt.count("-q")) return Report(Fetch(o, "GET", "/policy", "", &body), body);
        if (opt.count("-s")) {
            const std::string name = get("-n", "--name");
            const XPolicyType type = xsched::protocol::GetPolicyType(name);
            if (name.empty() || type <= kPolicyUnknown || type >= kPolicyMax) { std::fprintf(stderr, "xcli: unknown policy name '%s'\n", name.c_str()); return 1; }
            return Report(Fetch(o, "POST", "/policy?policy=" + std::to_string((int)type), "", &body), body);
        }
        return Usage();
    }
    if (cmd == "hint") {
        const std::string x = get("-x", "--xqueue"), pid = get("--pid", "--pid"), prio = get("-p", "--priority"), util = get("-u", "--utilization"), ts = get("-t", "--timeslice");
        const std::string handle = x.empty() ? "0" : std::to_string(std::strtoull(x.c_str(), nullptr, 0));
        std::string json;
        if (!prio.empty()) {
            if (x.empty()) { std::fprintf(stderr, "xcli: an XQueue handle is required for a priority hint\n"); return 1; }
            json = "{\"hint_type\": " + std::to_string((int)xsched::sched::kHintTypePriority) + ", \"handle\": " + handle + ", \"priority\": " + prio + "}";
        } else if (!util.empty()) {
            if (x.empty() && pid.empty()) { std::fprintf(stderr, "xcli: an XQueue handle or a pid is required for a utilization hint\n"); return 1; }
            json = "{\"hint_type\": " + std::to_string((int)xsched::sched::kHintTypeUtilization) + ", \"handle\": " + handle + ", \"pid\": " + (pid.empty() ? "0" : pid) +
                   ", \"utilization\": " + util + "}";
        } else if (!ts.empty()) {
            json = "{\"hint_type\": " + std::to_string((int)xsched::sched::kHintTypeTimeslice) + ", \"timeslice\": " + ts + "}";
        } else return Usage();
        std::string body;
        return Report(Fetch(o, "POST", "/hint", json, &body), body);
    }
    return Usage();
}
