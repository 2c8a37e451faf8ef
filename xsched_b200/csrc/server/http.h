// A small HTTP/1.1 endpoint and the little JSON the control routes need — enough for `xcli` and for scripts
// (urllib, curl).  One thread accepts, each request is read, answered and its connection closed.  The reference
// serves the same routes with cpp-httplib and jsoncpp (service/server/src/server.cpp:28-39,228-544); neither is
// vendored, so the subset used by the routes lives here: request line, headers, Content-Length body, query string
// and form-encoded parameters, flat JSON objects with integer / string / boolean members.
#pragma once
#include <atomic>
#include <cstdint>
#include <functional>
#include <map>
#include <string>
#include <thread>
#include <vector>

namespace xsched::service {

struct HttpRequest {
    std::string method, path, body;
    std::map<std::string, std::string> params;       // query string and application/x-www-form-urlencoded body
    bool Has(const std::string &k) const { return params.count(k) != 0; }
    const std::string &Get(const std::string &k) const { static const std::string none; auto it = params.find(k); return it == params.end() ? none : it->second; }
};

struct HttpResponse {
    int status = 200;
    std::string body;                                 // application/json
};

using HttpHandler = std::function<void(const HttpRequest &, HttpResponse &)>;

class HttpServer {
public:
    ~HttpServer() { Stop(); }
    /// Routes are matched on method and on the path up to an optional trailing ":param" segment, e.g.
    /// Route("GET", "/xqueue/", h) answers GET /xqueue/<anything>; the remainder is passed as params["_tail"].
    void Route(const std::string &method, const std::string &prefix, bool takes_tail, HttpHandler h);
    /// Binds addr:port (port 0 = pick one) and starts the accepting thread.  Returns the port, 0 on failure.
    uint16_t Start(const std::string &addr, uint16_t port);
    void Stop();
private:
    struct Entry { std::string method, prefix; bool tail; HttpHandler handler; };
    void Serve(int fd);
    std::vector<Entry> routes_;
    std::thread thread_;
    std::atomic<bool> stop_{false};
    int listen_fd_ = -1;
};

/// Flat JSON object -> members as strings (numbers and booleans in their literal form, strings unescaped).
/// Nested values are not supported; returns false on anything it cannot read.
bool ParseFlatJson(const std::string &text, std::map<std::string, std::string> *out);
std::string JsonEscape(const std::string &s);

/// Minimal blocking client (used by xcli): one request, returns the status (0 = could not connect) and the body.
int HttpCall(const std::string &addr, uint16_t port, const std::string &method, const std::string &target, const std::string &body, std::string *response);

} // namespace xsched::service
