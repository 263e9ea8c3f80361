#include "openai_server.hpp"

#include <cmath>
#include <arpa/inet.h>
#include <cerrno>
#include <chrono>
#include <cstring>
#include <netinet/in.h>
#include <poll.h>
#include <stdexcept>
#include <sys/socket.h>
#include <unistd.h>

namespace pocket {

namespace {

bool send_all(int fd, const std::string& s) {
  size_t off = 0;
  while (off < s.size()) {
    const ssize_t n = ::send(fd, s.data() + off, s.size() - off, MSG_NOSIGNAL);
    if (n <= 0) {
      if (errno == EINTR) continue;
      return false;
    }
    off += size_t(n);
  }
  return true;
}

const char* reason(int status) {
  switch (status) {
    case 200: return "OK";
    case 400: return "Bad Request";
    case 404: return "Not Found";
    case 405: return "Method Not Allowed";
    case 413: return "Payload Too Large";
    case 501: return "Not Implemented";
    case 503: return "Service Unavailable";
    default: return "Internal Server Error";
  }
}

std::string http_response(int status, const std::string& type, const std::string& body) {
  return "HTTP/1.1 " + std::to_string(status) + " " + reason(status) + "\r\nContent-Type: " + type +
         "\r\nContent-Length: " + std::to_string(body.size()) + "\r\nConnection: close\r\n\r\n" + body;
}

Json error_body(const std::string& msg, const std::string& type) {
  Json e = Json::object();
  e.set("message", msg);
  e.set("type", type);
  Json o = Json::object();
  o.set("error", e);
  return o;
}

double now_s() { return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count(); }

}  // namespace

OpenAIServer::OpenAIServer(InferenceEngine& engine, OpenAIServerOptions opt, SchedulerOptions sched)
    : eng_(engine), opt_(std::move(opt)) {
  sched_ = std::make_unique<BatchScheduler>(eng_, sched);
  if (!opt_.sidecar_argv.empty()) sidecar_ = std::make_unique<PythonSidecar>(opt_.sidecar_argv);
}

OpenAIServer::~OpenAIServer() { stop(); }

void OpenAIServer::start() {
  listen_fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
  if (listen_fd_ < 0) throw std::runtime_error(std::string("socket: ") + strerror(errno));
  int one = 1;
  setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_port = htons(uint16_t(opt_.port));
  if (inet_pton(AF_INET, opt_.host.c_str(), &addr.sin_addr) != 1) throw std::runtime_error("bad listen address " + opt_.host);
  if (::bind(listen_fd_, reinterpret_cast<sockaddr*>(&addr), sizeof addr) != 0 || ::listen(listen_fd_, 64) != 0) {
    const std::string why = strerror(errno);
    ::close(listen_fd_);
    listen_fd_ = -1;
    throw std::runtime_error("cannot listen on " + opt_.host + ":" + std::to_string(opt_.port) + ": " + why);
  }
  socklen_t len = sizeof addr;
  getsockname(listen_fd_, reinterpret_cast<sockaddr*>(&addr), &len);
  port_ = ntohs(addr.sin_port);
  stop_ = false;
  thread_ = std::thread([this] { accept_loop(); });
}

void OpenAIServer::stop() {
  if (stop_.exchange(true)) {
    if (thread_.joinable()) thread_.join();
    return;
  }
  // wake the accept thread, let it leave, and only then give the descriptor back: closing it first would let the
  // thread poll or accept on a number that another socket of the process may already have been given
  if (listen_fd_ >= 0) ::shutdown(listen_fd_, SHUT_RDWR);
  if (thread_.joinable()) thread_.join();
  if (listen_fd_ >= 0) {
    ::close(listen_fd_);
    listen_fd_ = -1;
  }
  {
    // no new connections from here on; unblock the ones that sit in recv / send
    std::lock_guard<std::mutex> lock(conn_mu_);
    for (int fd : conn_fds_) ::shutdown(fd, SHUT_RDWR);
  }
  if (sched_) sched_->stop();           // requests waiting for a result wake up as cancelled
  {
    std::unique_lock<std::mutex> lock(conn_mu_);
    conn_cv_.wait_for(lock, std::chrono::seconds(10), [this] { return live_connections_ == 0; });
  }
  if (sidecar_) sidecar_->shutdown();
}

void OpenAIServer::accept_loop() {
  while (!stop_) {
    pollfd pfd{listen_fd_, POLLIN, 0};
    const int rc = poll(&pfd, 1, 200);
    if (rc <= 0) continue;
    const int fd = ::accept(listen_fd_, nullptr, nullptr);
    if (fd < 0) continue;
    {
      std::lock_guard<std::mutex> lock(conn_mu_);
      conn_fds_.insert(fd);
      ++live_connections_;
    }
    std::thread([this, fd] {
      serve_connection(fd);
      std::lock_guard<std::mutex> lock(conn_mu_);
      conn_fds_.erase(fd);
      ::close(fd);                      // under the lock: stop() never shuts down a descriptor that was reused
      --live_connections_;
      conn_cv_.notify_all();
    }).detach();
  }
}

void OpenAIServer::serve_connection(int fd) {
  std::string buf;
  size_t header_end = std::string::npos;
  char tmp[16384];
  const double t0 = now_s();
  while (header_end == std::string::npos) {
    pollfd pfd{fd, POLLIN, 0};
    if (now_s() - t0 > 30) return;                      // a header that trickles in is given up on as well
    if (poll(&pfd, 1, 1000) <= 0) { if (now_s() - t0 > 10) return; continue; }
    const ssize_t n = ::recv(fd, tmp, sizeof tmp, 0);
    if (n <= 0) return;
    buf.append(tmp, size_t(n));
    header_end = buf.find("\r\n\r\n");
    if (buf.size() > (1u << 20) && header_end == std::string::npos) { send_all(fd, http_response(413, "text/plain", "headers too large")); return; }
  }
  const std::string head = buf.substr(0, header_end);
  const size_t sp1 = head.find(' '), sp2 = head.find(' ', sp1 + 1);
  if (sp1 == std::string::npos || sp2 == std::string::npos) { send_all(fd, http_response(400, "text/plain", "bad request line")); return; }
  const std::string method = head.substr(0, sp1);
  std::string path = head.substr(sp1 + 1, sp2 - sp1 - 1);
  const size_t q = path.find('?');
  if (q != std::string::npos) path.resize(q);
  size_t content_length = 0;
  {
    std::string lower = head;
    for (auto& c : lower) c = char(tolower(c));
    const size_t p = lower.find("content-length:");
    if (p != std::string::npos) {
      // digits only (after optional blanks), up to the end of the line: "-5", "abc" and "12x" are refused, not guessed
      size_t q = p + 15;
      while (q < lower.size() && (lower[q] == ' ' || lower[q] == '\t')) ++q;
      const size_t first = q;
      unsigned long long v = 0;
      bool ok = true;
      while (q < lower.size() && lower[q] >= '0' && lower[q] <= '9') {
        if (v > (1ull << 40)) { ok = false; break; }
        v = v * 10 + unsigned(lower[q] - '0');
        ++q;
      }
      while (ok && q < lower.size() && (lower[q] == ' ' || lower[q] == '\t')) ++q;
      ok = ok && q > first && (q >= lower.size() || lower[q] == '\r' || lower[q] == '\n');
      if (!ok && q > first && v > (1ull << 40)) { send_all(fd, http_response(413, "text/plain", "body too large")); return; }
      if (!ok) { send_all(fd, http_response(400, "text/plain", "bad content-length")); return; }
      content_length = size_t(v);
    }
  }
  if (content_length > (64u << 20)) { send_all(fd, http_response(413, "text/plain", "body too large")); return; }
  std::string body = buf.substr(header_end + 4);
  while (body.size() < content_length) {
    pollfd pfd{fd, POLLIN, 0};
    if (poll(&pfd, 1, 5000) <= 0) return;
    const ssize_t n = ::recv(fd, tmp, sizeof tmp, 0);
    if (n <= 0) return;
    body.append(tmp, size_t(n));
  }
  Reply r{500, "application/json", ""};
  try {
    bool streamed = false;
    if (method == "POST" && (path == "/v1/chat/completions" || path == "/v1/completions")) {
      const Json j = Json::parse(body);
      if (j["stream"].as_bool(false)) {
        r = completion(j, path == "/v1/chat/completions", fd);
        streamed = r.status == 0;
      } else {
        r = completion(j, path == "/v1/chat/completions", -1);
      }
    } else {
      r = handle(method, path, body);
    }
    if (!streamed) send_all(fd, http_response(r.status, r.content_type, r.body));
  } catch (const std::exception& e) {
    send_all(fd, http_response(400, "application/json", error_body(e.what(), "invalid_request_error").dump()));
  }
  ++served_;
}

OpenAIServer::Reply OpenAIServer::handle(const std::string& method, const std::string& path, const std::string& body) {
  if (path == "/health" || path == "/alive" || path == "/ready") {
    if (method != "GET") return {405, "application/json", error_body("use GET", "invalid_request_error").dump()};
    const SchedulerStats st = sched_->stats();
    Json o = Json::object();
    o.set("status", "ok");
    o.set("queued", int64_t(st.queued));
    o.set("decoding", int64_t(st.decoding));
    o.set("completed", int64_t(st.completed));
    o.set("kv_blocks_total", int64_t(st.kv_blocks_total));
    o.set("sidecar", sidecar_ ? (sidecar_->ping() ? "ok" : "down") : "none");
    return {200, "application/json", o.dump()};
  }
  if (path == "/v1/models") {
    if (method != "GET") return {405, "application/json", error_body("use GET", "invalid_request_error").dump()};
    Json m = Json::object();
    m.set("id", opt_.model_name);
    m.set("object", "model");
    m.set("owned_by", "pocketllm");
    Json data = Json::array();
    data.push_back(m);
    Json o = Json::object();
    o.set("object", "list");
    o.set("data", data);
    return {200, "application/json", o.dump()};
  }
  if (path == "/v1/chat/completions" || path == "/v1/completions") {
    if (method != "POST") return {405, "application/json", error_body("use POST", "invalid_request_error").dump()};
    return completion(Json::parse(body), path == "/v1/chat/completions", -1);
  }
  return {404, "application/json", error_body("no route " + path, "invalid_request_error").dump()};
}

OpenAIServer::Reply OpenAIServer::completion(const Json& body, bool chat, int fd_for_stream) {
  // ---- prompt -> token ids
  std::vector<int32_t> prompt;
  const bool thinking = body["thinking"].as_bool(false);
  // every id must be a whole number the model has a row for: a kernel indexes tables with it
  const int64_t vocab = eng_.vocab_size();
  auto take_token = [&](const Json& t) {
    if (!t.is_number()) return false;
    const double d = t.as_double();
    if (!(d >= 0.0) || d > 2147483647.0 || d != std::floor(d)) return false;
    if (vocab > 0 && d >= double(vocab)) return false;
    prompt.push_back(int32_t(d));
    return true;
  };
  if (body.contains("prompt_token_ids")) {
    if (!body["prompt_token_ids"].is_array())
      return {400, "application/json", error_body("prompt_token_ids must be a list of token ids", "invalid_request_error").dump()};
    for (const Json& t : body["prompt_token_ids"].items())
      if (!take_token(t))
        return {400, "application/json", error_body("prompt_token_ids holds a value that is not a token id of this model", "invalid_request_error").dump()};
  } else {
    if (!sidecar_) return {501, "application/json", error_body("text prompts need the templating sidecar; send prompt_token_ids", "unsupported_feature").dump()};
    Json req = Json::object();
    req.set("op", "encode");
    req.set("family", opt_.chat_family);
    if (chat) {
      req.set("messages", body["messages"]);
      if (body.contains("tools")) req.set("tools", body["tools"]);
      req.set("thinking", thinking);
    } else {
      Json msg = Json::object();
      msg.set("role", "user");
      msg.set("content", body["prompt"]);
      Json msgs = Json::array();
      msgs.push_back(msg);
      req.set("messages", msgs);
    }
    const Json enc = sidecar_->call(req);
    if (!enc["ok"].as_bool(false)) return {400, "application/json", error_body(enc["error"].as_string(), "invalid_request_error").dump()};
    if (!enc.contains("token_ids")) return {501, "application/json", error_body("the sidecar has no tokenizer; send prompt_token_ids", "unsupported_feature").dump()};
    for (const Json& t : enc["token_ids"].items())
      if (!take_token(t))
        return {400, "application/json", error_body("the tokenizer produced an id outside this model's vocabulary", "invalid_request_error").dump()};
  }
  if (prompt.empty()) return {400, "application/json", error_body("empty prompt", "invalid_request_error").dump()};
  int max_new = opt_.default_max_tokens;
  if (body.contains("max_tokens") && !body["max_tokens"].is_null()) {
    const Json& m = body["max_tokens"];
    const double d = m.is_number() ? m.as_double() : -1.0;
    if (!(d >= 1.0) || d > 1.0e9 || d != std::floor(d))
      return {400, "application/json", error_body("max_tokens must be a whole number >= 1", "invalid_request_error").dump()};
    max_new = int(d);
  }
  if (int64_t(prompt.size()) + 1 > eng_.max_context())
    return {400, "application/json", error_body("prompt does not fit the context window", "invalid_request_error").dump()};

  const uint64_t rid = next_id_++;
  const std::string id = (chat ? "chatcmpl-" : "cmpl-") + std::to_string(rid);
  const uint64_t sid = sched_->submit(prompt, max_new, true);
  SchedulerResult res;
  if (!sched_->wait(sid, res, -1) || res.finish_reason == "error")
    return {503, "application/json", error_body(res.error.empty() ? "generation failed" : res.error, "backend_unavailable").dump()};
  std::vector<int32_t> toks = res.tokens;
  const bool hit_eos = !toks.empty() && eng_.is_eos(toks.back());
  if (hit_eos) toks.pop_back();

  // ---- token ids -> text (when the sidecar can)
  Json tok_json = Json::array();
  for (int32_t t : toks) tok_json.push_back(Json(int64_t(t)));
  Json message = Json::object();
  message.set("role", "assistant");
  message.set("content", Json());
  std::string text;
  if (sidecar_) {
    try {
      Json req = Json::object();
      req.set("op", "decode");
      req.set("family", opt_.chat_family);
      req.set("token_ids", tok_json);
      req.set("thinking", thinking);
      const Json dec = sidecar_->call(req);
      if (dec["ok"].as_bool(false)) {
        text = dec["text"].as_string();
        if (dec.contains("message")) message = dec["message"];
        else message.set("content", text);
      }
    } catch (const std::exception&) {
    }
  }
  Json usage = Json::object();
  usage.set("prompt_tokens", int64_t(prompt.size()));
  usage.set("completion_tokens", int64_t(toks.size()));
  usage.set("total_tokens", int64_t(prompt.size() + toks.size()));
  Json timings = Json::object();
  timings.set("queue_seconds", res.queue_seconds);
  timings.set("prefill_seconds", res.prefill_seconds);
  timings.set("decode_seconds", res.decode_seconds);
  Json choice = Json::object();
  choice.set("index", 0);
  choice.set("finish_reason", hit_eos ? "stop" : res.finish_reason);
  choice.set("token_ids", tok_json);
  if (chat) choice.set("message", message);
  else choice.set("text", text);
  Json out = Json::object();
  out.set("id", id);
  out.set("object", chat ? "chat.completion" : "text_completion");
  out.set("model", opt_.model_name);
  Json choices = Json::array();
  choices.push_back(choice);
  out.set("choices", choices);
  out.set("usage", usage);
  out.set("timings", timings);
  if (fd_for_stream < 0) return {200, "application/json", out.dump()};

  // ---- server-sent events: one chunk with the whole completion, then [DONE] (generation is not incremental here)
  std::string head = "HTTP/1.1 200 OK\r\nContent-Type: text/event-stream\r\nCache-Control: no-cache\r\nConnection: close\r\n\r\n";
  Json delta = Json::object();
  delta.set("role", "assistant");
  delta.set("content", text);
  Json ch = Json::object();
  ch.set("index", 0);
  ch.set("delta", delta);
  ch.set("token_ids", tok_json);
  ch.set("finish_reason", hit_eos ? "stop" : res.finish_reason);
  Json chunk = Json::object();
  chunk.set("id", id);
  chunk.set("object", "chat.completion.chunk");
  chunk.set("model", opt_.model_name);
  Json chs = Json::array();
  chs.push_back(ch);
  chunk.set("choices", chs);
  send_all(fd_for_stream, head + "data: " + chunk.dump() + "\n\ndata: [DONE]\n\n");
  return {0, "", ""};
}

}  // namespace pocket
