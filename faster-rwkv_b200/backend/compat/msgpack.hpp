// Minimal stand-in for msgpack-c, written for this repository: just the API surface the reference's
// model.cpp, tensor.cpp, kernels/default/init_model.cpp and tokenizer.cpp use (unpack -> object ->
// as<T>(), object(value, zone) constructors, pack(ostream, nested containers)).  msgpack-c itself is a
// FetchContent dependency of the reference (CMakeLists.txt:156-163) and is not available offline.
// The whole buffer is parsed into a tree of nodes; binary payloads are copied.
#pragma once
#include <cstdint>
#include <cstring>
#include <algorithm>
#include <iomanip>
#include <iostream>
#include <sstream>
#include <map>
#include <memory>
#include <optional>
#include <ostream>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <unordered_map>
#include <utility>
#include <vector>

namespace msgpack {

struct zone {};

class object;
namespace detail {
struct node {
  enum kind_t { NIL, BOOL, INT, UINT, FLOAT, STR, BIN, ARRAY, MAP } kind = NIL;
  bool b = false;
  int64_t i = 0;
  uint64_t u = 0;
  double f = 0;
  std::string s;  // STR and BIN payload
  std::vector<object> arr;
  std::vector<std::pair<object, object>> map;
};
template <typename T> struct is_vector : std::false_type {};
template <typename T, typename A> struct is_vector<std::vector<T, A>> : std::true_type {};
template <typename T> struct is_map : std::false_type {};
template <typename K, typename V, typename... R> struct is_map<std::map<K, V, R...>> : std::true_type {};
template <typename K, typename V, typename... R> struct is_map<std::unordered_map<K, V, R...>> : std::true_type {};
}  // namespace detail

class type_error : public std::runtime_error {
public:
  type_error() : std::runtime_error("msgpack: type error") {}
};

class object {
public:
  object() : n_(std::make_shared<detail::node>()) {}
  object(const char *s, zone &) : object() { n_->kind = detail::node::STR; n_->s = s; }
  object(const std::string &s, zone &) : object() { n_->kind = detail::node::STR; n_->s = s; }
  object(const std::vector<char> &bin, zone &) : object() {
    n_->kind = detail::node::BIN;
    n_->s.assign(bin.begin(), bin.end());
  }
  template <typename I, typename = std::enable_if_t<std::is_integral_v<I>>>
  object(const std::vector<I> &v, zone &) : object() {
    n_->kind = detail::node::ARRAY;
    for (auto x : v) {
      object e;
      e.n_->kind = detail::node::INT;
      e.n_->i = static_cast<int64_t>(x);
      n_->arr.push_back(e);
    }
  }
  detail::node &node() { return *n_; }
  const detail::node &node() const { return *n_; }

  template <typename T> T as() const {
    T out;
    convert(out);
    return out;
  }
  template <typename T> void convert(T &out) const { conv(out); }

private:
  std::shared_ptr<detail::node> n_;

  void conv(object &o) const { o = *this; }
  void conv(bool &o) const {
    if (n_->kind != detail::node::BOOL) throw type_error();
    o = n_->b;
  }
  void conv(std::string &o) const {
    if (n_->kind != detail::node::STR && n_->kind != detail::node::BIN) throw type_error();
    o = n_->s;
  }
  void conv(float &o) const { double d; conv(d); o = static_cast<float>(d); }
  void conv(double &o) const {
    if (n_->kind == detail::node::FLOAT) o = n_->f;
    else if (n_->kind == detail::node::INT) o = static_cast<double>(n_->i);
    else if (n_->kind == detail::node::UINT) o = static_cast<double>(n_->u);
    else throw type_error();
  }
  template <typename I, typename = std::enable_if_t<std::is_integral_v<I> && !std::is_same_v<I, bool> &&
                                                    !std::is_same_v<I, char>>>
  void conv(I &o) const {
    if (n_->kind == detail::node::INT) o = static_cast<I>(n_->i);
    else if (n_->kind == detail::node::UINT) o = static_cast<I>(n_->u);
    else throw type_error();
  }
  void conv(std::vector<char> &o) const {
    if (n_->kind != detail::node::BIN && n_->kind != detail::node::STR) throw type_error();
    o.assign(n_->s.begin(), n_->s.end());
  }
  template <typename T> void conv(std::vector<T> &o) const {
    if (n_->kind != detail::node::ARRAY) throw type_error();
    o.clear();
    o.reserve(n_->arr.size());
    for (const auto &e : n_->arr) o.push_back(e.template as<T>());
  }
  template <typename M> void conv_map(M &o) const {
    if (n_->kind != detail::node::MAP) throw type_error();
    o.clear();
    for (const auto &kv : n_->map)
      o[kv.first.template as<typename M::key_type>()] = kv.second.template as<typename M::mapped_type>();
  }
  template <typename K, typename V, typename... R> void conv(std::map<K, V, R...> &o) const { conv_map(o); }
  template <typename K, typename V, typename... R> void conv(std::unordered_map<K, V, R...> &o) const { conv_map(o); }
};

class object_handle {
public:
  explicit object_handle(object o) : o_(std::move(o)) {}
  const object &get() const { return o_; }
  const object *operator->() const { return &o_; }
  const object &operator*() const { return o_; }

private:
  object o_;
};

namespace detail {
class parser {
public:
  parser(const char *d, size_t n) : p_(reinterpret_cast<const uint8_t *>(d)), end_(p_ + n) {}
  object parse() {
    object o;
    node &n = o.node();
    const uint8_t t = byte();
    if (t <= 0x7f) { n.kind = node::UINT; n.u = t; }
    else if (t <= 0x8f) map(n, t & 0x0f);
    else if (t <= 0x9f) array(n, t & 0x0f);
    else if (t <= 0xbf) str(n, t & 0x1f, node::STR);
    else if (t >= 0xe0) { n.kind = node::INT; n.i = static_cast<int8_t>(t); }
    else switch (t) {
      case 0xc0: n.kind = node::NIL; break;
      case 0xc2: n.kind = node::BOOL; n.b = false; break;
      case 0xc3: n.kind = node::BOOL; n.b = true; break;
      case 0xc4: str(n, be(1), node::BIN); break;
      case 0xc5: str(n, be(2), node::BIN); break;
      case 0xc6: str(n, be(4), node::BIN); break;
      case 0xc7: { size_t len = be(1); need(len + 1); p_ += len + 1; break; }
      case 0xc8: { size_t len = be(2); need(len + 1); p_ += len + 1; break; }
      case 0xc9: { size_t len = be(4); need(len + 1); p_ += len + 1; break; }
      case 0xca: { uint32_t v = static_cast<uint32_t>(be(4)); float f; std::memcpy(&f, &v, 4); n.kind = node::FLOAT; n.f = f; break; }
      case 0xcb: { uint64_t v = be(8); double f; std::memcpy(&f, &v, 8); n.kind = node::FLOAT; n.f = f; break; }
      case 0xcc: n.kind = node::UINT; n.u = be(1); break;
      case 0xcd: n.kind = node::UINT; n.u = be(2); break;
      case 0xce: n.kind = node::UINT; n.u = be(4); break;
      case 0xcf: n.kind = node::UINT; n.u = be(8); break;
      case 0xd0: n.kind = node::INT; n.i = static_cast<int8_t>(be(1)); break;
      case 0xd1: n.kind = node::INT; n.i = static_cast<int16_t>(be(2)); break;
      case 0xd2: n.kind = node::INT; n.i = static_cast<int32_t>(be(4)); break;
      case 0xd3: n.kind = node::INT; n.i = static_cast<int64_t>(be(8)); break;
      case 0xd4: need(2); p_ += 2; break;
      case 0xd5: need(3); p_ += 3; break;
      case 0xd6: need(5); p_ += 5; break;
      case 0xd7: need(9); p_ += 9; break;
      case 0xd8: need(17); p_ += 17; break;
      case 0xd9: str(n, be(1), node::STR); break;
      case 0xda: str(n, be(2), node::STR); break;
      case 0xdb: str(n, be(4), node::STR); break;
      case 0xdc: array(n, be(2)); break;
      case 0xdd: array(n, be(4)); break;
      case 0xde: map(n, be(2)); break;
      case 0xdf: map(n, be(4)); break;
      default: throw std::runtime_error("msgpack: bad type byte");
    }
    return o;
  }

private:
  const uint8_t *p_, *end_;
  void need(size_t n) const {
    if (static_cast<size_t>(end_ - p_) < n) throw std::runtime_error("msgpack: truncated input");
  }
  uint8_t byte() { need(1); return *p_++; }
  uint64_t be(int n) {
    need(n);
    uint64_t v = 0;
    for (int i = 0; i < n; ++i) v = (v << 8) | *p_++;
    return v;
  }
  void str(node &n, size_t len, node::kind_t k) {
    need(len);
    n.kind = k;
    n.s.assign(reinterpret_cast<const char *>(p_), len);
    p_ += len;
  }
  void array(node &n, size_t cnt) {
    n.kind = node::ARRAY;
    n.arr.reserve(cnt);
    for (size_t i = 0; i < cnt; ++i) n.arr.push_back(parse());
  }
  void map(node &n, size_t cnt) {
    n.kind = node::MAP;
    n.map.reserve(cnt);
    for (size_t i = 0; i < cnt; ++i) {
      object k = parse();
      object v = parse();
      n.map.emplace_back(std::move(k), std::move(v));
    }
  }
};

inline void put_be(std::ostream &os, uint64_t v, int n) {
  for (int i = n - 1; i >= 0; --i) os.put(static_cast<char>((v >> (8 * i)) & 0xff));
}
inline void put_len(std::ostream &os, size_t n, uint8_t fix, uint8_t fixmax, uint8_t t16, uint8_t t32) {
  if (n <= fixmax) os.put(static_cast<char>(fix | n));
  else if (n <= 0xffff) { os.put(static_cast<char>(t16)); put_be(os, n, 2); }
  else { os.put(static_cast<char>(t32)); put_be(os, n, 4); }
}
inline void pack_int(std::ostream &os, int64_t v) {
  if (v >= 0 && v <= 0x7f) os.put(static_cast<char>(v));
  else if (v < 0 && v >= -32) os.put(static_cast<char>(v));
  else if (v >= 0) { os.put(static_cast<char>(0xcf)); put_be(os, static_cast<uint64_t>(v), 8); }
  else { os.put(static_cast<char>(0xd3)); put_be(os, static_cast<uint64_t>(v), 8); }
}
inline void pack_str(std::ostream &os, const std::string &s) {
  if (s.size() <= 31) os.put(static_cast<char>(0xa0 | s.size()));
  else if (s.size() <= 0xff) { os.put(static_cast<char>(0xd9)); put_be(os, s.size(), 1); }
  else if (s.size() <= 0xffff) { os.put(static_cast<char>(0xda)); put_be(os, s.size(), 2); }
  else { os.put(static_cast<char>(0xdb)); put_be(os, s.size(), 4); }
  os.write(s.data(), static_cast<std::streamsize>(s.size()));
}
inline void pack_bin(std::ostream &os, const char *d, size_t n) {
  if (n <= 0xff) { os.put(static_cast<char>(0xc4)); put_be(os, n, 1); }
  else if (n <= 0xffff) { os.put(static_cast<char>(0xc5)); put_be(os, n, 2); }
  else { os.put(static_cast<char>(0xc6)); put_be(os, n, 4); }
  os.write(d, static_cast<std::streamsize>(n));
}

inline void pack_value(std::ostream &os, const object &o);
inline void pack_value(std::ostream &os, const std::string &s) { pack_str(os, s); }
inline void pack_value(std::ostream &os, const char *s) { pack_str(os, s); }
inline void pack_value(std::ostream &os, float f) { uint32_t v; std::memcpy(&v, &f, 4); os.put(static_cast<char>(0xca)); put_be(os, v, 4); }
inline void pack_value(std::ostream &os, double f) { uint64_t v; std::memcpy(&v, &f, 8); os.put(static_cast<char>(0xcb)); put_be(os, v, 8); }
inline void pack_value(std::ostream &os, bool b) { os.put(static_cast<char>(b ? 0xc3 : 0xc2)); }
template <typename I, typename = std::enable_if_t<std::is_integral_v<I> && !std::is_same_v<I, bool>>>
inline void pack_value(std::ostream &os, I v) { pack_int(os, static_cast<int64_t>(v)); }
inline void pack_value(std::ostream &os, const std::vector<char> &v) { pack_bin(os, v.data(), v.size()); }
template <typename T> inline void pack_value(std::ostream &os, const std::vector<T> &v);
template <typename K, typename V, typename... R> inline void pack_value(std::ostream &os, const std::map<K, V, R...> &m);
template <typename K, typename V, typename... R> inline void pack_value(std::ostream &os, const std::unordered_map<K, V, R...> &m);

template <typename T> inline void pack_value(std::ostream &os, const std::vector<T> &v) {
  put_len(os, v.size(), 0x90, 15, 0xdc, 0xdd);
  for (const auto &e : v) pack_value(os, e);
}
template <typename M> inline void pack_map(std::ostream &os, const M &m) {
  put_len(os, m.size(), 0x80, 15, 0xde, 0xdf);
  for (const auto &kv : m) { pack_value(os, kv.first); pack_value(os, kv.second); }
}
template <typename K, typename V, typename... R> inline void pack_value(std::ostream &os, const std::map<K, V, R...> &m) { pack_map(os, m); }
template <typename K, typename V, typename... R> inline void pack_value(std::ostream &os, const std::unordered_map<K, V, R...> &m) { pack_map(os, m); }

inline void pack_value(std::ostream &os, const object &o) {
  const node &n = o.node();
  switch (n.kind) {
    case node::NIL: os.put(static_cast<char>(0xc0)); break;
    case node::BOOL: pack_value(os, n.b); break;
    case node::INT: pack_int(os, n.i); break;
    case node::UINT: if (n.u <= 0x7fffffffffffffffull) pack_int(os, static_cast<int64_t>(n.u)); else { os.put(static_cast<char>(0xcf)); put_be(os, n.u, 8); } break;
    case node::FLOAT: pack_value(os, n.f); break;
    case node::STR: pack_str(os, n.s); break;
    case node::BIN: pack_bin(os, n.s.data(), n.s.size()); break;
    case node::ARRAY: put_len(os, n.arr.size(), 0x90, 15, 0xdc, 0xdd); for (const auto &e : n.arr) pack_value(os, e); break;
    case node::MAP: put_len(os, n.map.size(), 0x80, 15, 0xde, 0xdf); for (const auto &kv : n.map) { pack_value(os, kv.first); pack_value(os, kv.second); } break;
  }
}
}  // namespace detail

inline object_handle unpack(const char *data, size_t len) {
  detail::parser p(data, len);
  return object_handle(p.parse());
}

template <typename Stream, typename T> inline void pack(Stream &os, const T &v) { detail::pack_value(os, v); }

}  // namespace msgpack
