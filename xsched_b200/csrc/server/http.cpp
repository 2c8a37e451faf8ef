#include "server/http.h"

#include <cerrno>
#include <cstring>
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

namespace xsched::service {
namespace {

std::string UrlDecode(const std::string &s) {
    std::string out;
    for (size_t i = 0; i < s.size(); ++i) {
        if (s[i] == '+') out += ' ';
        else if (s[i] == '%' && i + 2 < s.size() + 0 && isxdigit((unsigned char)s[i + 1]) && isxdigit((unsigned char)s[i + 2])) {
            out += (char)std::stoi(s.substr(i + 1, 2), nullptr, 16);
            i += 2;
        } else out += s[i];
    }
    return out;
}

void ParseParams(const std::string &text, std::map<std::string, std::string> *out) {
    size_t pos = 0;
    while (pos < text.size()) {
        size_t amp = text.find('&', pos);
        if (amp == std::string::npos) amp = text.size();
        const std::string item = text.substr(pos, amp - pos);
        const size_t eq = item.find('=');
        if (!item.empty()) (*out)[UrlDecode(item.substr(0, eq))] = eq == std::string::npos ? "" : UrlDecode(item.substr(eq + 1));
        pos = amp + 1;
    }
}

bool SendAll(int fd, const std::string &data) {
    size_t off = 0;
    while (off < data.size()) {
        const ssize_t n = ::send(fd, data.data() + off, data.size() - off, MSG_NOSIGNAL);
        if (n <= 0) { if (errno == EINTR) continue; return false; }
        off += (size_t)n;
    }
    return true;
}

// Reads until the header block and Content-Length bytes of body are in `buf` (bounded: 1 MiB, 5 s).
bool ReadMessage(int fd, std::string *head, std::string *body) {
    std::string buf;
    size_t header_end = std::string::npos, want_body = 0;
    char chunk[4096];
    while (buf.size() < (1u << 20)) {
        if (header_end != std::string::npos && buf.size() >= header_end + 4 + want_body) break;
        pollfd p{fd, POLLIN, 0};
        if (::poll(&p, 1, 5000) <= 0) return false;
        const ssize_t n = ::recv(fd, chunk, sizeof(chunk), 0);
        if (n < 0 && errno == EINTR) continue;
        if (n <= 0) { if (header_end != std::string::npos && want_body == 0) break; if (header_end == std::string::npos) return false; break; }
        buf.append(chunk, (size_t)n);
        if (header_end == std::string::npos) {
            header_end = buf.find("\r\n\r\n");
            if (header_end != std::string::npos) {
                std::string lower = buf.substr(0, header_end);
                for (char &c : lower) c = (char)tolower((unsigned char)c);
                const size_t cl = lower.find("content-length:");
                if (cl != std::string::npos) want_body = (size_t)std::strtoull(lower.c_str() + cl + 15, nullptr, 10);
            }
        }
    }
    if (header_end == std::string::npos) return false;
    *head = buf.substr(0, header_end);
    *body = buf.substr(header_end + 4, want_body ? want_body : std::string::npos);
    return true;
}

const char *Reason(int status) {
    switch (status) { case 200: return "OK"; case 400: return "Bad Request"; case 404: return "Not Found"; case 405: return "Method Not Allowed"; default: return "Internal Server Error"; }
}

} // namespace

void HttpServer::Route(const std::string &method, const std::string &prefix, bool takes_tail, HttpHandler h) {
    routes_.push_back(Entry{method, prefix, takes_tail, std::move(h)});
}

uint16_t HttpServer::Start(const std::string &addr, uint16_t port) {
    listen_fd_ = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (listen_fd_ < 0) return 0;
    int one = 1;
    ::setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in sa{};
    sa.sin_family = AF_INET;
    sa.sin_port = htons(port);
    if (::inet_pton(AF_INET, addr.c_str(), &sa.sin_addr) != 1 || ::bind(listen_fd_, (sockaddr *)&sa, sizeof(sa)) != 0 || ::listen(listen_fd_, 16) != 0) {
        ::close(listen_fd_);
        listen_fd_ = -1;
        return 0;
    }
    socklen_t len = sizeof(sa);
    ::getsockname(listen_fd_, (sockaddr *)&sa, &len);
    thread_ = std::thread([this] {
        while (!stop_.load()) {
            pollfd p{listen_fd_, POLLIN, 0};
            if (::poll(&p, 1, 100) <= 0) continue;
            const int fd = ::accept4(listen_fd_, nullptr, nullptr, SOCK_CLOEXEC);
            if (fd < 0) continue;
            Serve(fd);
            ::close(fd);
        }
    });
    return ntohs(sa.sin_port);
}

void HttpServer::Stop() {
    stop_.store(true);
    if (thread_.joinable()) thread_.join();
    if (listen_fd_ >= 0) { ::close(listen_fd_); listen_fd_ = -1; }
}

void HttpServer::Serve(int fd) {
    std::string head, body;
    HttpResponse res;
    if (!ReadMessage(fd, &head, &body)) return;
    HttpRequest req;
    const size_t eol = head.find("\r\n");
    const std::string line = head.substr(0, eol);
    const size_t sp1 = line.find(' '), sp2 = line.rfind(' ');
    if (sp1 == std::string::npos || sp2 <= sp1) res.status = 400;
    else {
        req.method = line.substr(0, sp1);
        std::string target = line.substr(sp1 + 1, sp2 - sp1 - 1);
        const size_t q = target.find('?');
        if (q != std::string::npos) { ParseParams(target.substr(q + 1), &req.params); target.resize(q); }
        req.path = UrlDecode(target);
        req.body = body;
        std::string lower = head;
        for (char &c : lower) c = (char)tolower((unsigned char)c);
        if (lower.find("application/x-www-form-urlencoded") != std::string::npos) ParseParams(body, &req.params);
        bool path_known = false, served = false;
        for (const Entry &e : routes_) {
            const bool match = e.tail ? (req.path.size() > e.prefix.size() && req.path.compare(0, e.prefix.size(), e.prefix) == 0) : req.path == e.prefix;
            if (!match) continue;
            path_known = true;
            if (e.method != req.method) continue;
            if (e.tail) req.params["_tail"] = req.path.substr(e.prefix.size());
            e.handler(req, res);
            served = true;
            break;
        }
        if (!served) res.status = path_known ? 405 : 404;
    }
    std::string out = "HTTP/1.1 " + std::to_string(res.status) + " " + Reason(res.status) + "\r\nContent-Type: application/json\r\nContent-Length: " +
                      std::to_string(res.body.size()) + "\r\nConnection: close\r\n\r\n" + res.body;
    SendAll(fd, out);
}

bool ParseFlatJson(const std::string &t, std::map<std::string, std::string> *out) {
    size_t i = 0;
    auto ws = [&] { while (i < t.size() && isspace((unsigned char)t[i])) ++i; };
    auto str = [&](std::string *s) {
        if (i >= t.size() || t[i] != '"') return false;
        for (++i; i < t.size() && t[i] != '"'; ++i) {
            if (t[i] == '\\' && i + 1 < t.size()) {
                ++i;
                switch (t[i]) { case 'n': *s += '\n'; break; case 't': *s += '\t'; break; case 'r': *s += '\r'; break; default: *s += t[i]; }
            } else *s += t[i];
        }
        if (i >= t.size()) return false;
        ++i;
        return true;
    };
    ws();
    if (i >= t.size() || t[i] != '{') return false;
    ++i;
    ws();
    if (i < t.size() && t[i] == '}') return true;
    while (true) {
        ws();
        std::string key, val;
        if (!str(&key)) return false;
        ws();
        if (i >= t.size() || t[i] != ':') return false;
        ++i;
        ws();
        if (i < t.size() && t[i] == '"') { if (!str(&val)) return false; }
        else {
            const size_t b = i;
            while (i < t.size() && t[i] != ',' && t[i] != '}' && !isspace((unsigned char)t[i])) {
                if (t[i] == '{' || t[i] == '[') return false;
                ++i;
            }
            val = t.substr(b, i - b);
            if (val.empty()) return false;
        }
        (*out)[key] = val;
        ws();
        if (i < t.size() && t[i] == ',') { ++i; continue; }
        if (i < t.size() && t[i] == '}') return true;
        return false;
    }
}

std::string JsonEscape(const std::string &s) {
    std::string out;
    for (unsigned char c : s) {
        if (c == '"' || c == '\\') { out += '\\'; out += (char)c; }
        else if (c == '\n') out += "\\n";
        else if (c == '\t') out += "\\t";
        else if (c < 0x20) { char b[8]; std::snprintf(b, sizeof(b), "\\u%04x", c); out += b; }
        else out += (char)c;
    }
    return out;
}

int HttpCall(const std::string &addr, uint16_t port, const std::string &method, const std::string &target, const std::string &body, std::string *response) {
    const int fd = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd < 0) return 0;
    sockaddr_in sa{};
    sa.sin_family = AF_INET;
    sa.sin_port = htons(port);
    if (::inet_pton(AF_INET, addr.c_str(), &sa.sin_addr) != 1 || ::connect(fd, (sockaddr *)&sa, sizeof(sa)) != 0) { ::close(fd); return 0; }
    const std::string req = method + " " + target + " HTTP/1.1\r\nHost: " + addr + "\r\nContent-Type: application/json\r\nContent-Length: " +
                            std::to_string(body.size()) + "\r\nConnection: close\r\n\r\n" + body;
    int status = 0;
    std::string head, payload;
    if (SendAll(fd, req) && ReadMessage(fd, &head, &payload)) {
        const size_t sp = head.find(' ');
        if (sp != std::string::npos) status = std::atoi(head.c_str() + sp + 1);
        if (response) *response = payload;
    }
    ::close(fd);
    return status;
}

} // namespace xsched::service
