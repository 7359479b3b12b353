// ne-gateway: HTTP/1.1 gateway in front of a pool of engines, with prefill/decode (PD) routing and SSE pass-through.
//
//   ne-gateway [start|status|stop] --port 3001 [--host 0.0.0.0] [--ctrl-address http://h:p] [--ctrl-scope NAME] [--hybrid URL,...]
//              [--prefill URL,...] [--decode URL,...] [--model-alias alias=model ...] [--daemonize] [--pid-file PATH]
//
// Without a sub-command the gateway serves in the foreground.  `start` runs it as a daemon and records its pid under the runtime
// directory ($NANOENGINE_ROUTER_RUNTIME_DIR, default /tmp/nanoengine-router), `status` says whether that daemon is alive and prints
// its /status page, `stop` ends it.
//
// Routing.  Hybrid pool: round-robin reverse proxy.  PD pools (both non-empty): (1) POST the body to a prefill engine with
// stream=false and kv_transfer_params={"do_remote_decode":true}; (2) read kv_transfer_params.{migration,seq_id,first_token}
// from its JSON reply - if there is no migration but there are choices the request finished inside prefill and the reply
// is returned (as SSE when the caller asked to stream); (3) POST the original body with kv_transfer_params={migration,
// seq_id,first_token} and the caller's `stream` to a decode engine; (4) pass its bytes through (text/event-stream);
// (5) POST {prefill}/pd/free with the seq_id.  Upstream failures map to 502.  Discovery: every 5 s POST
// {ctrl}/list_entities; engines that appear are added to their role's pool, engines that vanish are removed.
//
// GET /status: uptime, engines per role, models, request counters, the control plane in use.  --ctrl-scope: only entities the
// control plane lists under that scope are taken (the scope is sent with the query and checked on every entity that names one).
//
// Parity: reference rust/src/router/mod.rs:11-231 (CLI, start / status / stop, daemonize, pid file), engine_manager.rs:8-68,100-105,
// 219-452 (pools, scope, discovery, stale removal, P/D pairing), http_server.rs:130-267 (PD forward), :475-483 (routes).
#include <arpa/inet.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <signal.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <functional>
#include <map>
#include <mutex>
#include <set>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

#include "json_lite.h"

static void logf(const char* lvl, const std::string& msg) {
  auto t = std::chrono::system_clock::to_time_t(std::chrono::system_clock::now());
  char buf[32]; strftime(buf, sizeof buf, "%H:%M:%S", localtime(&t));
  fprintf(stderr, "%s [%s] %s\n", buf, lvl, msg.c_str());
}

struct Url { std::string host; int port = 80; std::string base; };

static bool parse_url(const std::string& u, Url* out) {
  std::string s = u;
  if (s.rfind("http://", 0) == 0) s = s.substr(7);
  size_t slash = s.find('/');
  std::string hp = slash == std::string::npos ? s : s.substr(0, slash);
  out->base = slash == std::string::npos ? "" : s.substr(slash);
  while (!out->base.empty() && out->base.back() == '/') out->base.pop_back();
  size_t colon = hp.rfind(':');
  if (colon == std::string::npos) { out->host = hp; out->port = 80; }
  else { out->host = hp.substr(0, colon); out->port = atoi(hp.c_str() + colon + 1); }
  return !out->host.empty() && out->port > 0;
}

static int connect_to(const Url& u, int timeout_s = 10) {
  addrinfo hints{}, *res = nullptr;
  hints.ai_family = AF_INET; hints.ai_socktype = SOCK_STREAM;
  if (getaddrinfo(u.host.c_str(), std::to_string(u.port).c_str(), &hints, &res) != 0 || !res) return -1;
  int fd = socket(res->ai_family, res->ai_socktype, res->ai_protocol);
  if (fd >= 0) {
    timeval tv{timeout_s, 0};
    setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof tv);
    if (connect(fd, res->ai_addr, res->ai_addrlen) != 0) { close(fd); fd = -1; }
    else { int one = 1; setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one); }
  }
  freeaddrinfo(res);
  return fd;
}

static bool send_all(int fd, const char* p, size_t n) {
  while (n) { ssize_t k = send(fd, p, n, MSG_NOSIGNAL); if (k <= 0) return false; p += k; n -= (size_t)k; }
  return true;
}
static bool send_all(int fd, const std::string& s) { return send_all(fd, s.data(), s.size()); }

struct HttpMsg {
  std::string start;                              // request line or status line
  std::map<std::string, std::string> headers;     // lower-case names
  std::string body;
  int status() const { return start.size() > 12 ? atoi(start.c_str() + 9) : 0; }
};

static std::string lower(std::string s) { for (auto& c : s) c = (char)tolower((unsigned char)c); return s; }

// Reads the head of a message; leaves bytes past the head in `rest`.
static bool read_head(int fd, HttpMsg* m, std::string* rest) {
  std::string buf = *rest;
  char tmp[8192];
  size_t end;
  while ((end = buf.find("\r\n\r\n")) == std::string::npos) {
    if (buf.size() > (1u << 20)) return false;
    ssize_t k = recv(fd, tmp, sizeof tmp, 0);
    if (k <= 0) return false;
    buf.append(tmp, (size_t)k);
  }
  std::istringstream is(buf.substr(0, end));
  std::string line;
  std::getline(is, m->start);
  if (!m->start.empty() && m->start.back() == '\r') m->start.pop_back();
  while (std::getline(is, line)) {
    if (!line.empty() && line.back() == '\r') line.pop_back();
    size_t c = line.find(':');
    if (c == std::string::npos) continue;
    std::string v = line.substr(c + 1);
    while (!v.empty() && v.front() == ' ') v.erase(v.begin());
    m->headers[lower(line.substr(0, c))] = v;
  }
  *rest = buf.substr(end + 4);
  return true;
}

// Reads a body with Content-Length or chunked encoding (or until EOF) into m->body.
static bool read_body(int fd, HttpMsg* m, std::string* rest) {
  char tmp[16384];
  auto more = [&]() -> bool { ssize_t k = recv(fd, tmp, sizeof tmp, 0); if (k <= 0) return false; rest->append(tmp, (size_t)k); return true; };
  auto it = m->headers.find("content-length");
  if (it != m->headers.end()) {
    size_t n = (size_t)atoll(it->second.c_str());
    while (rest->size() < n) if (!more()) return false;
    m->body = rest->substr(0, n); *rest = rest->substr(n);
    return true;
  }
  auto te = m->headers.find("transfer-encoding");
  if (te != m->headers.end() && lower(te->second).find("chunked") != std::string::npos) {
    while (true) {
      size_t eol;
      while ((eol = rest->find("\r\n")) == std::string::npos) if (!more()) return false;
      size_t n = (size_t)strtoul(rest->substr(0, eol).c_str(), nullptr, 16);
      *rest = rest->substr(eol + 2);
      while (rest->size() < n + 2) if (!more()) return false;
      if (n == 0) { *rest = rest->substr(2); return true; }
      m->body.append(*rest, 0, n); *rest = rest->substr(n + 2);
    }
  }
  if (m->start.rfind("HTTP/", 0) == 0) { while (more()) {} m->body = *rest; rest->clear(); }   // response delimited by close
  return true;
}

static std::string make_request(const std::string& method, const Url& u, const std::string& path, const std::string& body,
                                const std::string& content_type = "application/json") {
  std::ostringstream o;
  o << method << " " << u.base << path << " HTTP/1.1\r\nHost: " << u.host << ":" << u.port << "\r\nConnection: close\r\n";
  if (!body.empty() || method == "POST") o << "Content-Type: " << content_type << "\r\nContent-Length: " << body.size() << "\r\n";
  o << "\r\n" << body;
  return o.str();
}

static bool http_call(const Url& u, const std::string& method, const std::string& path, const std::string& body, HttpMsg* resp, int timeout_s = 600) {
  int fd = connect_to(u);
  if (fd < 0) return false;
  timeval tv{timeout_s, 0}; setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof tv);
  bool ok = send_all(fd, make_request(method, u, path, body));
  std::string rest;
  ok = ok && read_head(fd, resp, &rest) && read_body(fd, resp, &rest);
  close(fd);
  return ok;
}

static void respond(int fd, int code, const std::string& body, const std::string& ctype = "application/json") {
  const char* reason = code == 200 ? "OK" : code == 404 ? "Not Found" : code == 400 ? "Bad Request" : code == 502 ? "Bad Gateway" : code == 503 ? "Service Unavailable" : "Error";
  std::ostringstream o;
  o << "HTTP/1.1 " << code << " " << reason << "\r\nContent-Type: " << ctype << "\r\nContent-Length: " << body.size() << "\r\nConnection: close\r\n\r\n" << body;
  send_all(fd, o.str());
}
static void respond_error(int fd, int code, const std::string& msg) {
  respond(fd, code, "{\"error\":{\"message\":" + jl::quote(msg) + ",\"type\":\"gateway_error\",\"code\":" + std::to_string(code) + "}}");
}

// ---- engine pools ---------------------------------------------------------------------------------
struct Engine { std::string id, url, role, model; bool from_ctrl = false; };

class Pools {
 public:
  void add(const Engine& e) {
    std::lock_guard<std::mutex> lk(mu_);
    for (auto& x : engines_) if (x.url == e.url && x.role == e.role) return;
    engines_.push_back(e);
    logf("info", "engine added: " + e.role + " " + e.url + (e.model.empty() ? "" : " model=" + e.model));
  }
  // Replace the control-plane view: add what is new, drop what disappeared ("heartbeat lost").
  void sync_from_ctrl(const std::vector<Engine>& seen) {
    std::lock_guard<std::mutex> lk(mu_);
    std::set<std::string> now;
    for (auto& e : seen) now.insert(e.role + "|" + e.url);
    for (auto it = engines_.begin(); it != engines_.end();) {
      if (it->from_ctrl && !now.count(it->role + "|" + it->url)) { logf("warn", "engine removed (heartbeat lost): " + it->url); it = engines_.erase(it); }
      else ++it;
    }
    for (auto& e : seen) {
      bool have = false;
      for (auto& x : engines_) if (x.url == e.url && x.role == e.role) have = true;
      if (!have) { engines_.push_back(e); logf("info", "engine discovered: " + e.role + " " + e.url); }
    }
  }
  bool pick(const std::string& role, const std::string& model, Engine* out) {
    std::lock_guard<std::mutex> lk(mu_);
    std::vector<const Engine*> c;
    for (auto& e : engines_) if (e.role == role && (model.empty() || e.model.empty() || e.model == model)) c.push_back(&e);
    if (c.empty()) return false;
    *out = *c[rr_[role]++ % c.size()];
    return true;
  }
  bool has(const std::string& role) { std::lock_guard<std::mutex> lk(mu_); for (auto& e : engines_) if (e.role == role) return true; return false; }
  std::vector<Engine> all() { std::lock_guard<std::mutex> lk(mu_); return engines_; }
 private:
  std::mutex mu_;
  std::vector<Engine> engines_;
  std::map<std::string, size_t> rr_;
};

static Pools g_pools;
static std::map<std::string, std::string> g_alias;
static std::atomic<bool> g_stop{false};
static std::atomic<long long> g_requests{0}, g_pd_requests{0}, g_failed{0};
static std::string g_ctrl, g_scope;
static int g_listen_fd = -1;
static const auto g_started = std::chrono::steady_clock::now();

static void discovery_loop(std::string ctrl) {
  Url cu;
  if (!parse_url(ctrl, &cu)) return;
  const std::string query = g_scope.empty() ? "{}" : "{\"scope\":" + jl::quote(g_scope) + "}";
  while (!g_stop) {
    HttpMsg r;
    if (http_call(cu, "POST", "/list_entities", query, &r, 5) && r.status() == 200) {
      // reply: {"entities":[{"id":..,"role":..,"host":..,"port":..,"model":..}, ...]}
      std::vector<Engine> seen;
      auto arr = jl::raw(r.body, "entities");
      if (arr && arr->size() > 2) {
        std::string_view a(*arr);
        size_t i = 1;
        while (i < a.size()) {
          i = jl::skip_ws(a, i);
          if (i >= a.size() || a[i] == ']') break;
          size_t e = jl::skip_value(a, i);
          if (e == std::string_view::npos) break;
          std::string_view obj = a.substr(i, e - i);
          Engine en; en.from_ctrl = true;
          if (auto v = jl::raw(obj, "id")) en.id = jl::unquote(*v);
          if (auto v = jl::raw(obj, "role")) en.role = jl::unquote(*v);
          if (auto v = jl::raw(obj, "model")) en.model = jl::unquote(*v);
          std::string host = "127.0.0.1"; int port = 0;
          if (auto v = jl::raw(obj, "host")) host = jl::unquote(*v);
          if (auto v = jl::raw(obj, "port")) port = atoi(v->c_str());
          if (auto v = jl::raw(obj, "url")) en.url = jl::unquote(*v); else en.url = "http://" + host + ":" + std::to_string(port);
          if (en.role.empty()) en.role = "hybrid";
          bool in_scope = true;
          if (!g_scope.empty()) if (auto v = jl::raw(obj, "scope")) in_scope = jl::unquote(*v) == g_scope;
          if (in_scope && (port > 0 || !en.url.empty())) seen.push_back(en);
          i = jl::skip_ws(a, e);
          if (i < a.size() && a[i] == ',') i++;
        }
      }
      g_pools.sync_from_ctrl(seen);
    }
    for (int k = 0; k < 50 && !g_stop; k++) std::this_thread::sleep_for(std::chrono::milliseconds(100));
  }
}

// Streams an upstream response to the client as it arrives.  Returns false if upstream could not be reached.
static bool proxy_stream(int cfd, const Url& u, const std::string& path, const std::string& body) {
  int ufd = connect_to(u);
  if (ufd < 0) return false;
  timeval tv{900, 0}; setsockopt(ufd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof tv);
  if (!send_all(ufd, make_request("POST", u, path, body))) { close(ufd); return false; }
  char tmp[16384];
  bool any = false;
  while (true) {
    ssize_t k = recv(ufd, tmp, sizeof tmp, 0);
    if (k <= 0) break;
    any = true;
    if (!send_all(cfd, tmp, (size_t)k)) break;     // client went away: stop reading, upstream sees the close
  }
  close(ufd);
  return any;
}

static std::string sse_from_completion(const std::string& json_body) {
  return "data: " + json_body + "\n\ndata: [DONE]\n\n";
}

static void forward_pd(int cfd, const std::string& path, const std::string& body, const std::string& model) {
  Engine p, d;
  if (!g_pools.pick("prefill", model, &p) || !g_pools.pick("decode", model, &d)) { respond_error(cfd, 503, "no prefill/decode engine pair available"); return; }
  Url pu, du;
  if (!parse_url(p.url, &pu) || !parse_url(d.url, &du)) { respond_error(cfd, 502, "bad engine url"); return; }
  const bool want_stream = jl::is_true(body, "stream");
  std::string pbody = jl::with_member(jl::with_member(body, "stream", "false"), "kv_transfer_params", "{\"do_remote_decode\":true}");
  HttpMsg pr;
  if (!http_call(pu, "POST", path, pbody, &pr) || pr.status() != 200) { respond_error(cfd, 502, "prefill engine failed" + (pr.status() ? " with status " + std::to_string(pr.status()) : std::string())); return; }
  auto kv = jl::raw(pr.body, "kv_transfer_params");
  std::optional<std::string> mig, seq, first;
  if (kv) { mig = jl::raw(*kv, "migration"); seq = jl::raw(*kv, "seq_id"); first = jl::raw(*kv, "first_token"); }
  if (!mig || *mig == "null") {
    // finished inside prefill (EOS or one-token request): hand the reply through
    auto ch = jl::raw(pr.body, "choices");
    if (!ch) { respond_error(cfd, 502, "prefill reply carries neither a migration nor choices"); return; }
    if (want_stream) respond(cfd, 200, sse_from_completion(pr.body), "text/event-stream"); else respond(cfd, 200, pr.body);
    return;
  }
  std::string kvd = "{\"migration\":" + *mig + ",\"seq_id\":" + (seq ? *seq : "0") + ",\"first_token\":" + (first ? *first : "null") + "}";
  std::string dbody = jl::with_member(body, "kv_transfer_params", kvd);
  bool ok = proxy_stream(cfd, du, path, dbody);
  if (!ok) respond_error(cfd, 502, "decode engine unreachable");
  HttpMsg fr;
  http_call(pu, "POST", "/pd/free", "{\"seq_id\":" + (seq ? *seq : "0") + "}", &fr, 10);
}

static void handle(int cfd) {
  timeval tv{60, 0}; setsockopt(cfd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof tv);
  HttpMsg req; std::string rest;
  if (!read_head(cfd, &req, &rest) || !read_body(cfd, &req, &rest)) { close(cfd); return; }
  std::istringstream rl(req.start);
  std::string method, path; rl >> method >> path;
  if (method == "GET" && path == "/health") {
    auto all = g_pools.all();
    respond(cfd, all.empty() ? 503 : 200, "{\"status\":\"" + std::string(all.empty() ? "no engines" : "ok") + "\",\"engines\":" + std::to_string(all.size()) + "}");
  } else if (method == "GET" && path == "/status") {
    int nh = 0, np = 0, nd = 0;
    std::set<std::string> names;
    for (auto& e : g_pools.all()) {
      (e.role == "prefill" ? np : e.role == "decode" ? nd : nh)++;
      if (!e.model.empty()) names.insert(e.model);
    }
    std::string models = "[";
    for (auto& n : names) models += std::string(models.size() > 1 ? "," : "") + jl::quote(n);
    const long long up = std::chrono::duration_cast<std::chrono::seconds>(std::chrono::steady_clock::now() - g_started).count();
    respond(cfd, 200, "{\"status\":\"" + std::string(nh + np + nd ? "ok" : "no engines") + "\",\"pid\":" + std::to_string(getpid()) + ",\"uptime_s\":" +
                          std::to_string(up) + ",\"engines\":{\"hybrid\":" + std::to_string(nh) + ",\"prefill\":" + std::to_string(np) + ",\"decode\":" +
                          std::to_string(nd) + "},\"pd_routing\":" + (np && nd ? "true" : "false") + ",\"models\":" + models + "],\"requests\":{\"total\":" +
                          std::to_string(g_requests.load()) + ",\"pd\":" + std::to_string(g_pd_requests.load()) + ",\"failed\":" +
                          std::to_string(g_failed.load()) + "},\"ctrl_address\":" + jl::quote(g_ctrl) + ",\"ctrl_scope\":" + jl::quote(g_scope) + "}");
  } else if (method == "GET" && path == "/v1/models") {
    std::set<std::string> names;
    for (auto& e : g_pools.all()) if (!e.model.empty()) names.insert(e.model);
    for (auto& a : g_alias) names.insert(a.first);
    std::string o = "{\"object\":\"list\",\"data\":[";
    bool first = true;
    for (auto& n : names) { o += std::string(first ? "" : ",") + "{\"id\":" + jl::quote(n) + ",\"object\":\"model\",\"owned_by\":\"nanoengine_b200\"}"; first = false; }
    respond(cfd, 200, o + "]}");
  } else if (method == "GET" && path == "/engines") {
    std::string o = "[";
    bool first = true;
    for (auto& e : g_pools.all()) { o += std::string(first ? "" : ",") + "{\"role\":" + jl::quote(e.role) + ",\"url\":" + jl::quote(e.url) + ",\"model\":" + jl::quote(e.model) + "}"; first = false; }
    respond(cfd, 200, o + "]");
  } else if (method == "POST" && (path == "/v1/chat/completions" || path == "/v1/completions" || path == "/v1/messages" || path == "/v1/messages/count_tokens")) {
    std::string body = req.body, model;
    if (auto m = jl::raw(body, "model")) {
      model = jl::unquote(*m);
      auto a = g_alias.find(model);
      if (a != g_alias.end()) { model = a->second; body = jl::with_member(body, "model", jl::quote(model)); }
    }
    const bool pd = g_pools.has("prefill") && g_pools.has("decode") && path != "/v1/messages/count_tokens";
    g_requests++;
    if (pd) { g_pd_requests++; forward_pd(cfd, path, body, model); }
    else {
      Engine e; Url u;
      if (!g_pools.pick("hybrid", model, &e) && !g_pools.pick("decode", model, &e) && !g_pools.pick("prefill", model, &e)) { g_failed++; respond_error(cfd, 503, "no engine available"); }
      else if (!parse_url(e.url, &u) || !proxy_stream(cfd, u, path, body)) { g_failed++; respond_error(cfd, 502, "engine unreachable: " + e.url); }
    }
  } else {
    respond_error(cfd, 404, "unknown route " + method + " " + path);
  }
  shutdown(cfd, SHUT_RDWR);
  close(cfd);
}

static std::vector<std::string> split(const std::string& s, char c) {
  std::vector<std::string> out; std::string cur; std::istringstream is(s);
  while (std::getline(is, cur, c)) if (!cur.empty()) out.push_back(cur);
  return out;
}

static std::string runtime_dir() {
  const char* d = getenv("NANOENGINE_ROUTER_RUNTIME_DIR");
  return d && *d ? d : "/tmp/nanoengine-router";
}
static long read_pid(const std::string& file) {
  std::ifstream f(file);
  long p = 0;
  return (f >> p) && p > 0 ? p : 0;
}
static bool alive(long pid) { return pid > 0 && kill((pid_t)pid, 0) == 0; }
static void on_term(int) {
  g_stop = true;
  if (g_listen_fd >= 0) shutdown(g_listen_fd, SHUT_RDWR);      // wakes the accept loop
}

int main(int argc, char** argv) {
  std::string host = "0.0.0.0", ctrl, pid_file, cmd;
  int port = 3001; bool daemonize = false;
  for (int i = 1; i < argc; i++) {
    std::string a = argv[i];
    auto next = [&]() -> std::string { return i + 1 < argc ? argv[++i] : ""; };
    if (i == 1 && (a == "start" || a == "status" || a == "stop")) cmd = a;
    else if (a == "--port") port = atoi(next().c_str());
    else if (a == "--host") host = next();
    else if (a == "--ctrl-address") ctrl = next();
    else if (a == "--ctrl-scope") g_scope = next();
    else if (a == "--hybrid" || a == "--prefill" || a == "--decode") { for (auto& u : split(next(), ',')) g_pools.add({"", u, a.substr(2), "", false}); }
    else if (a == "--model-alias") { auto kv = split(next(), '='); if (kv.size() == 2) g_alias[kv[0]] = kv[1]; }
    else if (a == "--daemonize") daemonize = true;
    else if (a == "--pid-file") pid_file = next();
    else if (a == "--help") { printf("usage: ne-gateway [start|status|stop] --port P [--host H] [--ctrl-address URL] [--ctrl-scope S] [--hybrid URLS] [--prefill URLS] [--decode URLS] [--model-alias a=b] [--daemonize] [--pid-file F]\n"); return 0; }
    else { fprintf(stderr, "unknown flag %s\n", a.c_str()); return 2; }
  }
  g_ctrl = ctrl;
  if (!cmd.empty()) {
    mkdir(runtime_dir().c_str(), 0755);
    if (pid_file.empty()) pid_file = runtime_dir() + "/ne-gateway.pid";
    const long pid = read_pid(pid_file);
    if (cmd == "status") {
      if (!alive(pid)) { printf("ne-gateway is not running\n"); return 3; }
      printf("ne-gateway is running (pid=%ld)\n", pid);
      Url self; self.host = "127.0.0.1"; self.port = port;
      HttpMsg r;
      if (http_call(self, "GET", "/status", "", &r, 3) && r.status() == 200) printf("%s\n", r.body.c_str());
      else printf("status page: unavailable on port %d\n", port);
      return 0;
    }
    if (cmd == "stop") {
      if (!alive(pid)) { printf("ne-gateway is not running\n"); unlink(pid_file.c_str()); return 0; }
      kill((pid_t)pid, SIGTERM);
      for (int k = 0; k < 50 && alive(pid); k++) usleep(100 * 1000);
      if (alive(pid)) { printf("ne-gateway (pid=%ld) did not stop\n", pid); return 1; }
      unlink(pid_file.c_str());
      printf("ne-gateway stopped (pid=%ld)\n", pid);
      return 0;
    }
    if (alive(pid)) { printf("ne-gateway is already running (pid=%ld)\n", pid); return 0; }
    daemonize = true;                                     // start
  }
  signal(SIGPIPE, SIG_IGN);
  signal(SIGTERM, on_term);
  signal(SIGINT, on_term);
  if (daemonize) {
    pid_t p = fork();
    if (p < 0) return 1;
    if (p > 0) { if (cmd == "start") printf("ne-gateway started (pid=%d)\n", (int)p); return 0; }
    setsid();
    if (cmd == "start") {
      // the daemon keeps none of the caller's descriptors: its log goes to the runtime directory
      FILE* n = freopen("/dev/null", "r", stdin); (void)n;
      n = freopen("/dev/null", "w", stdout); (void)n;
      n = freopen((runtime_dir() + "/ne-gateway.log").c_str(), "a", stderr); (void)n;
    }
  }
  if (!pid_file.empty()) { std::ofstream f(pid_file); f << getpid() << "\n"; }
  int ls = socket(AF_INET, SOCK_STREAM, 0);
  g_listen_fd = ls;
  int one = 1; setsockopt(ls, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  sockaddr_in addr{}; addr.sin_family = AF_INET; addr.sin_port = htons((uint16_t)port);
  inet_pton(AF_INET, host.c_str(), &addr.sin_addr);
  if (bind(ls, (sockaddr*)&addr, sizeof addr) != 0 || listen(ls, 512) != 0) { perror("ne-gateway: bind/listen"); return 1; }
  logf("info", "ne-gateway listening on " + host + ":" + std::to_string(port));
  std::thread disc;
  if (!ctrl.empty()) disc = std::thread(discovery_loop, ctrl);
  while (!g_stop) {
    int cfd = accept(ls, nullptr, nullptr);
    if (cfd < 0) { if (errno == EINTR && !g_stop) continue; break; }
    int nd = 1; setsockopt(cfd, IPPROTO_TCP, TCP_NODELAY, &nd, sizeof nd);
    std::thread(handle, cfd).detach();
  }
  g_stop = true;
  if (disc.joinable()) disc.join();
  if (!cmd.empty() && !pid_file.empty()) unlink(pid_file.c_str());
  return 0;
}
