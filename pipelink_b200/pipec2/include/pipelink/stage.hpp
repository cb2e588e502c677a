// <pipelink/stage.hpp>: the PL_* annotations a stage translation unit declares its contract with.
//
// `pipec2 pack stage.cu` compiles the unit twice. Once as the device payload, where every
// annotation below expands to nothing; and once with -DPIPELINK_EMIT as a host program, where each
// annotation is a static object that records one piece of the manifest and the `main` this header
// supplies prints the schema-3.0 manifest as JSON. Parameter sizes, alignments and member offsets
// come from the compiler that also builds the payload, so a manifest cannot drift from the
// struct it describes. The vocabulary follows the reference's device annotation set
// (docs/reference/annotations.md "Overview": PL_STAGE, PL_PARAMS / PL_NO_PARAMS /
// PL_PARAMS_OPAQUE, PL_ROLE, PL_EXPORT, PL_ENDPOINT, PL_CLAIM / PL_CLAIM_EX / PL_CLAIM_REGS,
// PL_TOPOLOGY, PL_VARIANT, PL_HINT); each annotation ends in `;`.
//
//   PL_STAGE("moe.load", "1.0.0");
//   PL_PARAMS(MoeLoadParams, a, b, sfa, sfb, g, counters);
//   PL_ROLE(load, moe_load_role, 1);
//   PL_ENDPOINT(operands, pl::endpoint(pl::produce, "load").space("smem")...);
//   PL_CLAIM(smem, pipelink_moe_operands, pl::per("pipelink_moe_depth", 35840), 1024);
//   PL_TOPOLOGY(pl::topology().cta_group(2).cluster(2, 1, 1).persistent());
#pragma once

#ifndef PIPELINK_EMIT

#define PL_STAGE(id, version) static_assert(true, "")
#define PL_PARAMS(T, ...) static_assert(true, "")
#define PL_PARAMS_OPAQUE(T) static_assert(true, "")
#define PL_NO_PARAMS() static_assert(true, "")
#define PL_ROLE(name, fn, warps) static_assert(true, "")
#define PL_EXPORT(name, fn) static_assert(true, "")
#define PL_CALL(channel, fn, direction, ...) static_assert(true, "")
#define PL_TYPE(...) static_assert(true, "")
#define PL_BINDING(...) static_assert(true, "")
#define PL_SITE(...) static_assert(true, "")
#define PL_EXPORT_TENSOR(...) static_assert(true, "")
#define PL_IMPORT_TENSOR(...) static_assert(true, "")
#define PL_DESCRIPTOR(T) static_assert(true, "")
#define PL_ENDPOINT(name, ...) static_assert(true, "")
#define PL_CLAIM(...) static_assert(true, "")
#define PL_CLAIM_EX(...) static_assert(true, "")
#define PL_CLAIM_SMEM(...) static_assert(true, "")
#define PL_CLAIM_WARPS(handle, role, warps, align) static_assert(true, "")
#define PL_CLAIM_REGS(...) static_assert(true, "")
#define PL_VARIANT_ENTRY(...) static_assert(true, "")
#define PL_TOPOLOGY(...) static_assert(true, "")
#define PL_VARIANT(...) static_assert(true, "")
#define PL_HINT(key, value) static_assert(true, "")

#else  // PIPELINK_EMIT: the host projection

// the manifest pass is plain C++: declarations of device functions parse, their bodies are left out
// by the unit (#ifndef PIPELINK_EMIT around the device code)
#ifndef __CUDACC__
#define __device__
#define __host__
#define __global__
#define __forceinline__ inline
#endif

#include "tensor_source.h"
#include <algorithm>
#include <array>
#include <cctype>
#include <optional>
#include <cstddef>
#include <cstdio>
#include <functional>
#include <tuple>
#include <initializer_list>
#include <map>
#include <memory>
#include <string>
#include <type_traits>
#include <utility>
#include <vector>

namespace pl {

// A JSON value: enough of one to print a manifest (objects print with sorted keys).
class json {
 public:
  enum Kind { Null, Bool, Int, Str, Arr, Obj };
  json() : kind_(Null) {}
  json(bool b) : kind_(Bool), i_(b) {}
  json(int v) : kind_(Int), i_(v) {}
  json(long v) : kind_(Int), i_(v) {}
  json(long long v) : kind_(Int), i_(v) {}
  json(unsigned long v) : kind_(Int), i_(static_cast<long long>(v)) {}
  json(const char* s) : kind_(Str), s_(s) {}
  json(const std::string& s) : kind_(Str), s_(s) {}
  static json array() { json j; j.kind_ = Arr; return j; }
  static json object() { json j; j.kind_ = Obj; return j; }
  template <class T>
  static json list(std::initializer_list<T> items) {
    json j = array();
    for (const T& item : items) j.push(json(item));
    return j;
  }
  json& push(json v) { kind_ = Arr; a_.push_back(std::move(v)); return *this; }
  json& operator[](const std::string& key) { kind_ = Obj; return o_[key]; }
  json& set(const std::string& key, json v) { (*this)[key] = std::move(v); return *this; }
  bool is_null() const { return kind_ == Null; }
  size_t size() const { return kind_ == Arr ? a_.size() : o_.size(); }
  json& at(size_t i) { return a_[i]; }
  const std::string& str() const { return s_; }
  std::string dump() const {
    switch (kind_) {
      case Null: return "null";
      case Bool: return i_ ? "true" : "false";
      case Int: return std::to_string(i_);
      case Str: return quote(s_);
      case Arr: {
        std::string out = "[";
        for (size_t i = 0; i < a_.size(); ++i) out += (i ? "," : "") + a_[i].dump();
        return out + "]";
      }
      default: {
        std::string out = "{";
        bool first = true;
        for (const auto& kv : o_) {
          out += (first ? "" : ",") + quote(kv.first) + ":" + kv.second.dump();
          first = false;
        }
        return out + "}";
      }
    }
  }

 private:
  static std::string quote(const std::string& s) {
    std::string out = "\"";
    for (char c : s) {
      if (c == '"' || c == '\\') { out += '\\'; out += c; }
      else if (c == '\n') out += "\\n";
      else out += c;
    }
    return out + "\"";
  }
  Kind kind_;
  long long i_ = 0;
  std::string s_;
  std::vector<json> a_;
  std::map<std::string, json> o_;
};

constexpr const char* produce = "produce";
constexpr const char* consume = "consume";

// extent of a claim: a constant, or a multiple of a link-time handle (a ring depth), or both
struct extent {
  long long constant = 0;
  std::map<std::string, long long> per_handle;
  extent operator+(const extent& o) const {
    extent e = *this;
    e.constant += o.constant;
    for (const auto& kv : o.per_handle) e.per_handle[kv.first] += kv.second;
    return e;
  }
  json to_json() const {
    json per = json::object();
    for (const auto& kv : per_handle) per[kv.first] = json(kv.second);
    json j = json::object();
    j["const"] = json(constant);
    j["per"] = per;
    return j;
  }
};
inline extent units(long long n) { extent e; e.constant = n; return e; }
inline extent per(const char* handle, long long n) { extent e; e.per_handle[handle] = n; return e; }

// depth of a ring: bound at link time through a handle, or fixed by the stage
struct depth {
  json j = json::object();
  static depth handle(const char* h) { depth d; d.j["handle"] = json(h); return d; }
  static depth fixed(int n) { depth d; d.j["fixed"] = json(n); return d; }
};

// one side of a barrier pair: who arrives, how many arrivals complete a phase, bytes credited
struct arrivals {
  json j = json::object();
  arrivals(const char* slots_handle, int count, const char* by_role, long long tx_bytes = 0) {
    j["slots"] = json(slots_handle);
    json a = json::object();
    a["count"] = json(count);
    a["by"] = json(by_role);
    j["arrive"] = a;
    j["tx_bytes"] = json(tx_bytes);
  }
};

// ---- the reference's spelling of the same declarations (docs/reference/annotations.md "Endpoints and
// protocols", "Topology and scheduling", "Resource claims"): a stage source written against its header
// packs here unchanged. Each type only gathers what it is given; the manifest text is made by to_json().
struct handle { const char* name; explicit handle(const char* n) : name(n) {} };
struct fixed { int n; explicit fixed(int value) : n(value) {} };

struct tree {            // a shape or stride tree: {128, 64} is [128, 64], {{64}} is [[64]]
  bool leaf;
  long long value = 0;
  std::vector<tree> kids;
  template <class I, typename std::enable_if<std::is_integral<I>::value, int>::type = 0>
  tree(I v) : leaf(true), value(static_cast<long long>(v)) {}
  tree(std::initializer_list<tree> k) : leaf(false), kids(k) {}
  json to_json() const {
    if (leaf) return json(value);
    json a = json::array();
    for (const tree& k : kids) a.push(k.to_json());
    return a;
  }
};
struct affine {          // pl::affine{shape, stride, elem_bits}[.swizzle(B, M, S)]
  tree shape, stride;
  int elem_bits, sw_b = 0, sw_m = 0, sw_s = 0;
  affine(std::initializer_list<tree> sh, std::initializer_list<tree> st, long long bits) : shape(sh), stride(st), elem_bits(static_cast<int>(bits)) {}
  affine& swizzle(int b, int m, int s_) { sw_b = b; sw_m = m; sw_s = s_; return *this; }
  json to_json() const {
    json l = json::object();
    l["encoding"] = json("pl-layout-v2");
    l["elem_bits"] = json(elem_bits);
    l["shape"] = shape.to_json();
    l["stride"] = stride.to_json();
    if (sw_b != 0) {
      json sw = json::object();
      sw["B"] = json(sw_b);
      sw["M"] = json(sw_m);
      sw["S"] = json(sw_s);
      l["swizzle"] = sw;
    }
    return l;
  }
};
struct tmem { int lanes_lo, lanes_hi, cols, elem_bits; };   // pl::tmem{lanes_lo, lanes_hi, cols, elem_bits}

struct arrive {          // pl::arrive{"role", 2} or pl::arrive{"role", "threads(role)"}
  std::string by;
  json count;
  arrive(const char* role, int n) : by(role), count(n) {}
  arrive(const char* role, const char* expression) : by(role), count(expression) {}
};
struct tile_t {};
constexpr tile_t tile{};      // pl::tile: the transaction bytes of a side are the bytes of the endpoint's tile
struct side {            // pl::side{slots handle, arrive, tx_bytes | pl::tile}
  std::string slots;
  arrive who;
  json tx;
  side(const char* slots_handle, const arrive& a, long long tx_bytes) : slots(slots_handle), who(a), tx(tx_bytes) {}
  side(const char* slots_handle, const arrive& a, tile_t) : slots(slots_handle), who(a), tx("tile") {}
  json to_json() const {
    json a = json::object();
    a["by"] = json(who.by);
    a["count"] = who.count;
    json j = json::object();
    j["slots"] = json(slots);
    j["arrive"] = a;
    j["tx_bytes"] = tx;
    return j;
  }
};
struct init {            // pl::init{owner, phase, materializer[, warp]}
  const char* owner;
  int phase;
  const char* materializer;
  int warp;
  init(const char* o, int ph, const char* m, int w = -1) : owner(o), phase(ph), materializer(m), warp(w) {}
};
struct mbarrier {        // pl::mbarrier{full, empty | std::nullopt, init[, release]}
  side full;
  bool has_empty;
  side empty;
  init start;
  std::string release;
  mbarrier(const side& f, const side& e, const init& i, const char* rel = "once-per-acquire")
      : full(f), has_empty(true), empty(e), start(i), release(rel) {}
  mbarrier(const side& f, std::nullopt_t, const init& i, const char* rel)
      : full(f), has_empty(false), empty(f), start(i), release(rel) {}
  json to_json() const {
    json i = json::object();
    if (start.owner != nullptr) i["owner"] = json(start.owner);
    i["phase"] = json(start.phase);
    i["materializer"] = json(start.materializer);
    if (start.warp >= 0) i["warp"] = json(start.warp);
    json p = json::object();
    p["kind"] = json("mbarrier");
    p["full"] = full.to_json();
    if (has_empty) p["empty"] = empty.to_json();
    p["init"] = i;
    p["release"] = json(release);
    return p;
  }
};
struct named_barrier { const char* id; int count; };        // pl::named_barrier{id handle, threads}
struct counter {                                             // pl::counter{slot[, release, acquire]}: grid scope
  const char* slot;
  const char* release;
  const char* acquire;
  counter(const char* s, const char* r = "red.release.gpu", const char* a = "ld.acquire.gpu") : slot(s), release(r), acquire(a) {}
};
struct counter_sys : counter {                               // the same at system scope
  counter_sys(const char* s, const char* r = "red.release.sys", const char* a = "ld.acquire.sys") : counter(s, r, a) {}
};

// PL_ENDPOINT's builder: one end of a channel (mbarrier ring, named barrier or counter)
class endpoint {
 public:
  // (direction, role): this header's own spelling; ("name", direction[, "role"]): the reference's
  endpoint(const char* first, const char* second, const char* role = nullptr) {
    const std::string a = first;
    if (a == produce || a == consume) {
      j_["direction"] = json(first);
      j_["owner_role"] = second ? json(second) : json();
    } else {
      j_["direction"] = json(second);
      j_["owner_role"] = role ? json(role) : json();
    }
    j_["binds"] = json::object();
  }
  endpoint& layout(const affine& a) { j_["layout"] = a.to_json(); return *this; }
  endpoint& layout(const tmem& t) { return layout_tmem(t.elem_bits, t.lanes_lo, t.lanes_hi, t.cols); }
  endpoint& ring(const handle& h, long long stage_stride_bytes) { return ring(depth::handle(h.name), stage_stride_bytes); }
  endpoint& ring(const fixed& f, long long stage_stride_bytes) { return ring(depth::fixed(f.n), stage_stride_bytes); }
  endpoint& protocol(const ::pl::mbarrier& m) { j_["protocol"] = m.to_json(); return *this; }
  endpoint& protocol(const named_barrier& b) {
    json p = json::object();
    p["kind"] = json("named_barrier");
    p["id"] = json(b.id);
    p["count"] = json(b.count);
    j_["protocol"] = p;
    return *this;
  }
  endpoint& protocol(const ::pl::counter& c) {
    json p = json::object();
    p["kind"] = json("counter");
    p["slot"] = json(c.slot);
    p["release"] = json(c.release);
    p["acquire"] = json(c.acquire);
    j_["protocol"] = p;
    return *this;
  }
  endpoint& exports(std::initializer_list<const char*> fns) {
    json e = json::array();
    for (const char* f : fns) e.push(json(f));
    j_["exports"] = e;
    return *this;
  }
  endpoint& space(const char* s) { j_["space"] = json(s); return *this; }
  endpoint& scope(const char* s) { j_["scope"] = json(s); return *this; }
  endpoint& proxy(const char* s) { j_["proxy"] = json(s); return *this; }
  endpoint& tile(const char* dtype, std::initializer_list<int> shape) {
    json t = json::object();
    t["dtype"] = json(dtype);
    t["shape"] = json::list(shape);
    j_["tile"] = t;
    return *this;
  }
  // shared-memory tile layout: per-mode shapes and strides in elements, optional swizzle <B, M, S>
  endpoint& layout_smem(int elem_bits, std::initializer_list<int> shape, std::initializer_list<int> stride,
                        int swizzle_b = 0, int swizzle_m = 0, int swizzle_s = 0) {
    json l = json::object();
    l["encoding"] = json("pl-layout-v2");
    l["elem_bits"] = json(elem_bits);
    json sh = json::array(), st = json::array();
    for (int v : shape) sh.push(json::list({v}));
    for (int v : stride) st.push(json::list({v}));
    l["shape"] = sh;
    l["stride"] = st;
    if (swizzle_b != 0) {
      json sw = json::object();
      sw["B"] = json(swizzle_b);
      sw["M"] = json(swizzle_m);
      sw["S"] = json(swizzle_s);
      l["swizzle"] = sw;
    }
    j_["layout"] = l;
    return *this;
  }
  // tensor-memory tile layout: a lane interval and a column count
  endpoint& layout_tmem(int elem_bits, int lane_begin, int lane_end, int cols) {
    json l = json::object();
    l["encoding"] = json("pl-layout-v2");
    l["elem_bits"] = json(elem_bits);
    l["lanes"] = json::list({lane_begin, lane_end});
    l["cols"] = json(cols);
    j_["layout"] = l;
    return *this;
  }
  endpoint& ring(const depth& d, long long stage_stride_bytes, long long payload_bytes = -1) {
    json r = json::object();
    r["depth"] = d.j;
    r["stage_stride_bytes"] = json(stage_stride_bytes);
    if (payload_bytes >= 0) r["payload_bytes"] = json(payload_bytes);
    j_["ring"] = r;
    return *this;
  }
  endpoint& mbarrier(const arrivals& full, const arrivals& empty, const char* init_owner) {
    json p = json::object();
    p["kind"] = json("mbarrier");
    p["full"] = full.j;
    p["empty"] = empty.j;
    json init = json::object();
    init["owner"] = json(init_owner);
    init["phase"] = json(0);
    init["materializer"] = json("dispatch");
    p["init"] = init;
    p["release"] = json("once-per-acquire");
    j_["protocol"] = p;
    return *this;
  }
  // a one-way signal: arrivals on a full barrier and nothing flowing back
  endpoint& mbarrier_full_only(const arrivals& full, const char* init_owner) {
    json p = json::object();
    p["kind"] = json("mbarrier");
    p["full"] = full.j;
    json init = json::object();
    init["owner"] = json(init_owner);
    init["phase"] = json(0);
    init["materializer"] = json("dispatch");
    p["init"] = init;
    p["release"] = json("once-per-acquire");
    j_["protocol"] = p;
    return *this;
  }
  endpoint& counter(const char* slot_handle, const char* release, const char* acquire) {
    json c = json::object();
    c["slot"] = json(slot_handle);
    c["release"] = json(release);
    c["acquire"] = json(acquire);
    json p = json::object();
    p["kind"] = json("counter");
    p["counter"] = c;
    j_["protocol"] = p;
    return *this;
  }
  endpoint& bind(const char* what, const char* handle) {
    if (j_["binds"].is_null()) j_["binds"] = json::object();
    j_["binds"][what] = json(handle);
    return *this;
  }
  json to_json(const char* name) const {
    json j = j_;
    j["name"] = json(name);
    return j;
  }

 private:
  json j_ = json::object();
};

// pl::signal_endpoint(name, direction[, role]): a barrier channel that carries completion and no data
inline endpoint signal_endpoint(const char* name, const char* direction, const char* role = nullptr) {
  endpoint e(name, direction, role);
  e.space("none").scope("cta").proxy("generic");
  return e;
}

struct launch {          // pl::launch{x_multiple_of, {max x, y, z}}
  int x_multiple_of;
  std::array<int, 3> max;
  launch(int multiple = 1, std::array<int, 3> m = {1, 1, 1}) : x_multiple_of(multiple), max(m) {}
};
struct dynamic_t {};
constexpr dynamic_t dynamic{};
struct cluster {         // pl::cluster{{x, y, z} | pl::dynamic, pl::launch{...}}
  bool is_dynamic;
  std::array<int, 3> compiled;
  launch at_launch;
  cluster(std::array<int, 3> c, const launch& l) : is_dynamic(false), compiled(c), at_launch(l) {}
  cluster(dynamic_t, const launch& l) : is_dynamic(true), compiled{1, 1, 1}, at_launch(l) {}
};

class topology {
 public:
  // pl::topology{cta_group, cluster, persistent, scheduler, multicast}: the reference's spelling
  topology(int group, const ::pl::cluster& c, bool is_persistent, const char* sched, std::initializer_list<const char*> multicast) {
    json mc = json::array();
    for (const char* m : multicast) mc.push(json(m));
    j_["multicast"] = mc;
    j_["persistent"] = json(is_persistent);
    j_["scheduler"] = json(sched);
    cta_group(group);
    json l = json::object();
    l["x_multiple_of"] = json(c.at_launch.x_multiple_of);
    l["max"] = json::list({c.at_launch.max[0], c.at_launch.max[1], c.at_launch.max[2]});
    json cl = json::object();
    cl["compiled"] = c.is_dynamic ? json("dynamic") : json::list({c.compiled[0], c.compiled[1], c.compiled[2]});
    cl["launch"] = l;
    j_["cluster"] = cl;
  }
  topology() {
    j_["multicast"] = json::array();
    j_["persistent"] = json(false);
    j_["scheduler"] = json("static");
    cta_group(1);
    cluster(1, 1, 1);
  }
  topology& cta_group(int n) {
    json g = json::object();
    g["fixed"] = json(n);
    j_["cta_group"] = g;
    return *this;
  }
  topology& cluster(int x, int y, int z) {
    json launch = json::object();
    launch["x_multiple_of"] = json(x);
    launch["max"] = json::list({x, y, z});
    json c = json::object();
    c["compiled"] = json::list({x, y, z});
    c["launch"] = launch;
    j_["cluster"] = c;
    return *this;
  }
  topology& persistent(bool on = true) { j_["persistent"] = json(on); return *this; }
  topology& scheduler(const char* s) { j_["scheduler"] = json(s); return *this; }
  const json& to_json() const { return j_; }

 private:
  json j_ = json::object();
};

// What the annotations of one translation unit add up to.
struct registry {
  json stage = json::object(), roles = json::object(), exports = json::object();
  json endpoints = json::array(), claims = json::array(), variants = json::array();
  json topology, params, descriptor, hints = json::object();
  json strong = json::array();
  json tensor_exports = json::array(), tensor_imports = json::array(), tensor_sites = json::array(), tensor_bindings = json::array();
  std::vector<std::pair<std::string, std::vector<long long>>> binding_values;   // PL_BINDING domains, by name
  std::vector<std::pair<std::string, std::string>> type_texts;                // PL_TYPE(T, members...): name -> definition
  std::vector<std::pair<std::string, int>> role_warps;   // every PL_ROLE, in order
  std::vector<std::string> warp_claimed;                // roles some warp claim names
  int errors = 0;
  static registry& get() { static registry r; return r; }
  void fail(const std::string& what) { std::fprintf(stderr, "stage.hpp: %s\n", what.c_str()); ++errors; }
};

struct reg_stage {
  reg_stage(const char* id, const char* version) {
    registry& r = registry::get();
    if (!r.stage.is_null() && r.stage.dump() != "{}") r.fail("more than one PL_STAGE");
    std::string prefix;
    for (const char* c = id; *c; ++c) prefix += (*c == '.' || *c == '-') ? '_' : *c;
    r.stage["id"] = json(id);
    r.stage["version"] = json(version);
    r.stage["symbol_prefix"] = json(prefix + "_");
  }
};

struct member { const char* name; size_t offset, size; };
// the name of a type as the compiler knows it, namespaces included ("pipelink_profile_consumer::InstructionParams")
template <class T>
std::string qualified_name(const char* as_written) {
  const std::string pretty = __PRETTY_FUNCTION__;       // "... [with T = ns::Type; ...]"
  const size_t at = pretty.find("T = ");
  if (at == std::string::npos) return as_written;
  size_t end = pretty.find_first_of(";]", at);
  return pretty.substr(at + 4, end - at - 4);
}

struct reg_descriptor {      // PL_DESCRIPTOR(T): the size and alignment of the stage's descriptor record
  reg_descriptor(size_t bytes, size_t align) {
    json d = json::object();
    d["bytes"] = json(static_cast<long long>(bytes));
    d["align"] = json(static_cast<long long>(align));
    registry::get().descriptor = d;
  }
};

struct reg_params {
  reg_params(const char* type, size_t bytes, size_t align, bool opaque, std::initializer_list<member> members) {
    registry& r = registry::get();
    if (!r.params.is_null()) r.fail("more than one PL_PARAMS / PL_NO_PARAMS / PL_PARAMS_OPAQUE");
    json p = json::object();
    p["type"] = json(type);
    p["bytes"] = json(static_cast<long long>(bytes));
    p["align"] = json(static_cast<long long>(align));
    p["opaque"] = json(opaque);
    json ms = json::array();
    for (const member& m : members) {
      json e = json::object();
      e["name"] = json(m.name);
      e["offset"] = json(static_cast<long long>(m.offset));
      e["bytes"] = json(static_cast<long long>(m.size));
      ms.push(e);
    }
    p["members"] = ms;
    r.params = p;
  }
};

struct reg_role {
  reg_role(const char* name, const char* entry, int warps) {
    registry& r = registry::get();
    json role = json::object();
    role["entry"] = json(entry);
    role["warps"] = json(warps);
    r.roles[name] = role;
    r.strong.push(json(entry));
    r.role_warps.push_back({name, warps});
  }
};

struct reg_export {
  reg_export(const char* name, const char* fn) {
    registry& r = registry::get();
    json e = json::object();
    e["symbol"] = json(fn);
    r.exports[name] = e;
    r.strong.push(json(fn));
  }
};

struct reg_endpoint {
  reg_endpoint(const char* name, const endpoint& e) { registry::get().endpoints.push(e.to_json(name)); }
};

struct reg_claim {
  reg_claim(const char* domain, const char* handle, const extent& e, int align, const char* key = nullptr, json value = json()) {
    json c = json::object();
    c["domain"] = json(domain);
    c["handle"] = json(handle);
    c["extent"] = e.to_json();
    c["align"] = json(align);
    c["lifetime"] = json("kernel");
    if (key != nullptr) c[key] = value;
    registry::get().claims.push(c);
  }
};

struct during { const char* tensor; const char* from; const char* to = nullptr; };
// pl::claim(handle, domain).extent(...).align(...).lifetime(...).at(...).roles({...}): the reference's builder
class claim {
 public:
  claim(const char* handle, const char* domain) : domain_(domain) {
    j_["handle"] = json(handle);
    j_["domain"] = json(domain);
    j_["extent"] = units(0).to_json();
    j_["align"] = json(1);
    j_["lifetime"] = json("kernel");
  }
  claim& extent(long long constant, std::initializer_list<std::pair<const char*, long long>> per_handle = {}) {
    ::pl::extent e = units(constant);
    for (const auto& kv : per_handle) e.per_handle[kv.first] += kv.second;
    j_["extent"] = e.to_json();
    return *this;
  }
  claim& align(int a) { j_["align"] = json(a); return *this; }
  claim& typed() { j_["_typed"] = json(true); return *this; }      // sized from a C++ type: the packer lists these last
  claim& lifetime(const char* l) { j_["lifetime"] = json(l); return *this; }
  claim& lifetime(const during& events) {       // held between two events of a tensor's life (pl::during{tensor, from, to})
    json l = json::object();
    l["tensor"] = json(events.tensor);
    l["from"] = json(events.from);
    l["to"] = events.to ? json(events.to) : json();
    j_["lifetime"] = l;
    return *this;
  }
  claim& lifetime() { return *this; }
  claim& at(long long base) { j_["absolute_base"] = json(base); return *this; }
  claim& roles(std::initializer_list<const char*> names) {
    json r = json::array();
    for (const char* n : names) { r.push(json(n)); roles_.push_back(n); }
    j_["roles"] = r;
    return *this;
  }
  const json& to_json() const { return j_; }
  void note_warps() const {          // a warp claim places the roles it names
    if (domain_ == "warp") for (const std::string& n : roles_) registry::get().warp_claimed.push_back(n);
  }

 private:
  json j_ = json::object();
  std::string domain_;
  std::vector<std::string> roles_;
};

struct reg_claim_any {
  static std::string bare(const char* token) {     // a stringified macro argument: quotes stay when the author wrote them
    std::string t = token;
    if (t.size() >= 2 && t.front() == '"' && t.back() == '"') t = t.substr(1, t.size() - 2);
    return t;
  }
  // PL_CLAIM(domain, handle, pl::units(n) | pl::per(...), align): this header's own spelling
  reg_claim_any(const char* domain, const char* handle, const ::pl::extent& e, int align) {
    reg_claim(bare(domain).c_str(), bare(handle).c_str(), e, align);
  }
  // PL_CLAIM("handle", "domain", extent, align[, lifetime[, role...]]): the reference's
  template <class... Roles>
  reg_claim_any(const char* handle, const char* domain, long long n, int align, const char* lifetime = "kernel", Roles... role_names) {
    claim c(bare(handle).c_str(), bare(domain).c_str());
    c.extent(n).align(align).lifetime(lifetime);
    if (sizeof...(Roles) > 0) c.roles({role_names...});
    c.note_warps();
    registry::get().claims.push(c.to_json());
  }
  explicit reg_claim_any(const claim& c) {   // PL_CLAIM_EX(pl::claim(...)...)
    c.note_warps();
    registry::get().claims.push(c.to_json());
  }
};

struct reg_warps {
  reg_warps(const char* handle, const char* role, int warps, int align) {
    json c = json::object();
    c["domain"] = json("warp");
    c["handle"] = json(handle);
    c["extent"] = units(warps).to_json();
    c["align"] = json(align);
    c["lifetime"] = json("kernel");
    c["roles"] = json::list({role});
    registry::get().warp_claimed.push_back(role);
    registry::get().claims.push(c);
  }
};

struct reg_regs {          // PL_CLAIM_REGS("handle", "reg_group", {values...}, "role"...)
  template <class... Roles>
  reg_regs(const char* handle, const char* group, std::initializer_list<int> values, Roles... role_names) {
    json c = json::object();
    c["domain"] = json("regs");
    c["handle"] = json(handle);
    c["reg_group"] = json(group);
    json roles = json::array();
    const char* names[] = {role_names..., nullptr};
    for (size_t i = 0; i < sizeof...(Roles); ++i) roles.push(json(names[i]));
    c["roles"] = roles;
    json vs = json::array();
    for (int v : values) vs.push(json(v));
    c["values"] = vs;
    registry::get().claims.push(c);
  }
};

struct reg_topology {
  explicit reg_topology(const topology& t) {
    registry& r = registry::get();
    if (!r.topology.is_null()) r.fail("more than one PL_TOPOLOGY");
    r.topology = t.to_json();
  }
};

struct reg_variant {       // PL_VARIANT(index, {{handle, value}, ...}); PL_VARIANT_ENTRY(index, {{...}}, fn)
  using key_list = std::initializer_list<std::pair<const char*, long long>>;
  static json key_of(key_list key) {
    json k = json::object();
    for (const auto& kv : key) k[kv.first] = json(kv.second);
    return k;
  }
  reg_variant(int index, json key) { push(index, key.is_null() ? json::object() : key, nullptr); }
  reg_variant(int index, key_list key) { push(index, key_of(key), nullptr); }
  // `text` is the stringified argument list: the entry's name is what follows its last comma
  reg_variant(int index, const char* text, key_list key, void (*)(const void*, unsigned)) {
    std::string t = text;
    t = t.substr(t.rfind(',') + 1);
    while (!t.empty() && t.front() == ' ') t.erase(0, 1);
    push(index, key_of(key), t.c_str());
    registry::get().strong.push(json(t));
  }
  static void push(int index, const json& key, const char* entry) {
    json v = json::object();
    v["index"] = json(index);
    v["key"] = key;
    if (entry != nullptr) v["entry"] = json(entry);
    registry::get().variants.push(v);
  }
};

struct reg_hint {
  reg_hint(const char* key, json value) { registry::get().hints[key] = std::move(value); }
};

inline int emit_main() {
  registry& r = registry::get();
  if (r.stage.dump() == "{}") r.fail("no PL_STAGE");
  if (r.params.is_null()) r.fail("no PL_PARAMS / PL_NO_PARAMS / PL_PARAMS_OPAQUE");
  if (r.topology.is_null()) r.topology = topology().to_json();
  if (r.errors != 0) return 1;
  // a role no claim places gets a warp claim of its own, handle pipelink_<role>_warps (what the reference's
  // pass adds: its hello-callable pipeline declares pipelink_call_warps for the role `call`)
  for (const auto& role : r.role_warps) {
    bool claimed = false;
    for (const std::string& who : r.warp_claimed) claimed = claimed || who == role.first;
    if (!claimed) {
      json c = json::object();
      c["domain"] = json("warp");
      c["handle"] = json("pipelink_" + role.first + "_warps");
      c["extent"] = units(role.second).to_json();
      c["align"] = json(1);
      c["lifetime"] = json("kernel");
      json roles = json::array();
      roles.push(json(role.first));
      c["roles"] = roles;
      r.claims.push(c);
    }
  }
  if (r.variants.dump() == "[]") reg_variant(0, json::object());
  json stage = r.stage;
  stage["entry_abi"] = json("v2");
  stage["entry_signature"] = json("void(const void* params, unsigned variant)");
  stage["roles"] = r.roles;
  stage["exports"] = r.exports;
  stage["variants"] = r.variants;
  if (!r.descriptor.is_null()) stage["descriptor"] = r.descriptor;
  json symbols = json::object();
  symbols["defined_strong"] = r.strong;
  json out = json::object();
  out["stage"] = stage;
  out["endpoints"] = r.endpoints;
  out["claims"] = r.claims;
  out["topology"] = r.topology;
  out["params"] = r.params;
  out["hints"] = r.hints;
  out["symbols"] = symbols;
  if (r.tensor_exports.size() + r.tensor_imports.size() + r.tensor_sites.size() + r.tensor_bindings.size() != 0) {
    // "all threads" of a site or a rendezvous: every thread of the site's role, 32 per warp
    auto threads_of = [&r](const std::string& role) {
      json set = json::array();
      for (const auto& rw : r.role_warps)
        if (rw.first == role)
          for (int t = 0; t < rw.second * 32; ++t) set.push(json(t));
      json who = json::object();
      who["set"] = set;
      return who;
    };
    for (size_t i = 0; i < r.tensor_sites.size(); ++i)
      if (r.tensor_sites.at(i)["participants"].is_null())
        r.tensor_sites.at(i)["participants"] = threads_of(r.tensor_sites.at(i)["role"].str());
    for (size_t i = 0; i < r.tensor_imports.size(); ++i) {
      json& imp = r.tensor_imports.at(i);
      std::string role;
      for (size_t k = 0; k < r.tensor_sites.size(); ++k)
        if (imp["sites"].size() != 0 && r.tensor_sites.at(k)["name"].str() == imp["sites"].at(0).str()) role = r.tensor_sites.at(k)["role"].str();
      for (size_t k = 0; k < imp["rendezvous"].size(); ++k)
        if (imp["rendezvous"].at(k)["cohort"].is_null()) imp["rendezvous"].at(k)["cohort"] = threads_of(role);
    }
    json tensor = json::object();
    tensor["version"] = json("tensor-v2");
    tensor["exports"] = r.tensor_exports;
    tensor["imports"] = r.tensor_imports;
    tensor["sites"] = r.tensor_sites;
    tensor["bindings"] = r.tensor_bindings;
    out["tensor"] = tensor;
  }
  std::puts(out.dump().c_str());
  return 0;
}

// C spellings of the types a call channel may carry (scalars, pointers to them, const): the link
// generates the trampoline from them, so the set is closed
template <class T> struct type_name;
#define PL_TYPE_NAME(T, spelled) template <> struct type_name<T> { static std::string get() { return spelled; } }
PL_TYPE_NAME(void, "void"); PL_TYPE_NAME(bool, "bool"); PL_TYPE_NAME(char, "char"); PL_TYPE_NAME(float, "float"); PL_TYPE_NAME(double, "double");
PL_TYPE_NAME(signed char, "int8_t"); PL_TYPE_NAME(unsigned char, "uint8_t"); PL_TYPE_NAME(short, "int16_t");
PL_TYPE_NAME(unsigned short, "uint16_t"); PL_TYPE_NAME(int, "int32_t"); PL_TYPE_NAME(unsigned, "uint32_t");
PL_TYPE_NAME(long, "int64_t"); PL_TYPE_NAME(unsigned long, "uint64_t"); PL_TYPE_NAME(long long, "int64_t");
PL_TYPE_NAME(unsigned long long, "uint64_t"); PL_TYPE_NAME(pipelink_tensor_source, "pipelink_tensor_source");
#undef PL_TYPE_NAME
template <class T> struct type_name<const T> { static std::string get() { return "const " + type_name<T>::get(); } };
template <class T> struct type_name<T*> { static std::string get() { return type_name<T>::get() + "*"; } };

template <class F> struct signature;
template <class R, class... A>
struct signature<R(A...)> {
  static std::string get() {
    std::string args;
    const std::string names[] = {type_name<A>::get()..., ""};
    for (size_t i = 0; i < sizeof...(A); ++i) args += (i ? ", " : "") + names[i];
    return type_name<R>::get() + "(" + args + ")";
  }
};

// one side of a call channel: the caller's trampoline (produce, from a role) or the provided function (consume)
// PL_TYPE(T, members...): the definitions of the registered structs a signature names, each behind an include
// guard of its own (<T IN CAPITALS>_DEFINED), in the order the signature names them
inline std::string type_definitions(const std::string& sig) {
  std::vector<std::pair<size_t, std::string>> found;
  for (const auto& t : registry::get().type_texts) {
    const size_t at = sig.find(t.first);
    if (at != std::string::npos) found.push_back({at, t.second});
  }
  std::sort(found.begin(), found.end());
  std::string out;
  for (const auto& f : found) out += f.second;
  return out;
}
struct reg_type {
  reg_type(const char* name, const char* members) {
    std::string guard;
    for (const char* c = name; *c; ++c) guard += static_cast<char>(std::toupper(static_cast<unsigned char>(*c)));
    guard += "_DEFINED";
    registry::get().type_texts.push_back({name, "#ifndef " + guard + "\n#define " + guard + "\nstruct " + name + " { " + members + " };\n#endif\n"});
  }
};

struct reg_type_if {   // registers the definition only when members were given
  reg_type_if(const char* name, const char* members) { if (*members) reg_type(name, members); }
};

struct reg_call {
  // one side of a call channel. The protocol carries the C declaration of this side's function, spelled
  // from its type: extern "C" __device__ float hello_scale(float);  (the digest is added by the packer)
  reg_call(const char* channel, const char* fn, const std::string& sig, const char* direction, const char* who,
           const char* export_name = nullptr) {
    const bool caller = std::string(direction) == produce;
    const size_t paren = sig.find('(');
    const std::string decl = type_definitions(sig) + "extern \"C\" __device__ " + sig.substr(0, paren) + " " + fn + sig.substr(paren) + ";";
    json proto = json::object();
    proto["kind"] = json("call");
    proto["export"] = json(caller ? (export_name ? export_name : channel) : who);
    proto["signature"] = json(sig);
    proto["decl"] = json(decl);
    json e = json::object();
    e["name"] = json(channel);
    e["direction"] = json(direction);
    e["owner_role"] = caller ? json(who) : json();
    e["space"] = json("reg");
    e["scope"] = json("cta");
    e["proxy"] = json("generic");
    json tile = json::object();
    tile["dtype"] = json("u64");
    tile["shape"] = json::list({1});
    e["tile"] = tile;
    json layout = json::object();
    layout["encoding"] = json("pl-layout-v2");
    layout["elem_bits"] = json(64);
    json one = json::array();
    one.push(json::list({1}));
    layout["shape"] = one;
    layout["stride"] = one;
    e["layout"] = layout;
    e["protocol"] = proto;
    e["binds"] = json::object();
    registry& r = registry::get();
    r.endpoints.push(e);
    if (!caller) {      // the provided side restates its declaration in the stage's export record
      if (r.exports[who].is_null()) r.exports[who] = json::object();
      r.exports[who]["symbol"] = json(fn);
      r.exports[who]["decl"] = json(decl);
    }
  }
};

// ---------------------------------------------------------------------------------------------------
// Tensor annotations (docs/reference/tensor-imports.md): PL_BINDING, PL_SITE, PL_EXPORT_TENSOR,
// PL_IMPORT_TENSOR. A map (where an export keeps each element; which thread wants which element) is
// written as a C++ lambda over named coordinates and bound values. The projection finds its
// integer-affine form from the origin of the domain and one step along every input and checks that form
// at every point of the full domain; a map that is not affine (an address swizzle) is solved as XOR-linear
// in the bits of its inputs. Either is printed in the manifest's expression language
// (["add", ["coord", "n"], ["toint", ["bind", "tmem_base"]]]); a map of neither family is refused.
struct all_threads_t {};
constexpr all_threads_t all_threads{};
struct coord { const char* name; int lo, hi; };
struct bound {                      // the value of a binding inside a map
  long long value;
  operator long long() const { return value; }
};
struct bind {
  const char* name; const char* sort;
  bind(const char* n, const char* s) : name(n), sort(s) {}
};
struct values {
  const char* name; const char* sort; std::vector<long long> items;
  values(const char* n, const char* s, std::initializer_list<long long> v) : name(n), sort(s), items(v) {}
};
struct strings : std::vector<std::string> {
  strings(std::initializer_list<const char*> v) { for (const char* x : v) push_back(x); }
  json to_json() const { json a = json::array(); for (const auto& x : *this) a.push(json(x)); return a; }
};
using guarantees = strings;
struct sync { int generations, capacity; };
struct lend {                       // field order: the reference's aggregate (stage.hpp:65-70 there), which sources brace-initialise
  const char* name; const char* domain; int extent, align;
  const char* scope; const char* binding; const char* handle;
  std::optional<int> base; const char* owner; const char* from; const char* to;
  std::optional<::pl::sync> barrier_sync = std::nullopt;
  json to_json() const {
    json j = json::object(), life = json::object(), where = json::object();
    life["from"] = json(from);
    life["to"] = json(to);
    where["base"] = base ? json(*base) : json();
    where["handle"] = handle ? json(handle) : json();
    j["name"] = json(name);
    j["domain"] = json(domain);
    j["extent"] = json(extent);
    j["align"] = json(align);
    j["scope"] = json(scope);
    j["binding"] = json(binding);
    j["owner"] = json(owner);
    j["lifetime"] = life;
    j["location"] = where;
    if (barrier_sync) {
      json sy = json::object();
      sy["generations"] = json(barrier_sync->generations);
      sy["capacity"] = json(barrier_sync->capacity);
      j["sync"] = sy;
    } else {
      j["sync"] = json();
    }
    return j;
  }
};
using lends = std::initializer_list<lend>;
inline json lends_json(lends all) { json a = json::array(); for (const lend& l : all) a.push(l.to_json()); return a; }
// the common lends by kind: shared-memory bytes at a link-time handle, registers of every thread, words of the
// caller's register frame, per-warp metadata words, a CTA barrier id with the generations the hand-off may use
constexpr lend smem(const char* name, int extent, int align, const char* handle, const char* owner, const char* from, const char* to) {
  return {name, "smem", extent, align, "cta", "relocatable", handle, std::nullopt, owner, from, to};
}
constexpr lend regs(const char* name, int extent, const char* handle, const char* owner, const char* from, const char* to) {
  return {name, "reg", extent, 1, "thread", "fixed", handle, std::nullopt, owner, from, to};
}
constexpr lend frame(const char* name, int words, const char* handle, const char* owner, const char* from, const char* to) {
  return {name, "reg", words, 1, "thread", "caller_frame", handle, std::nullopt, owner, from, to};
}
constexpr lend metadata(const char* name, int extent, const char* handle, const char* owner, const char* from, const char* to) {
  return {name, "metadata", extent, 1, "warp", "fixed", handle, std::nullopt, owner, from, to};
}
constexpr lend cta_barrier(const char* name, int base, const char* owner, const char* from, const char* to, ::pl::sync s) {
  return {name, "barrier", 1, 1, "cta", "fixed", nullptr, base, owner, from, to, s};
}
struct arg { const char* name; const char* meaning; };
using args = std::initializer_list<arg>;
struct readiness { const char* after; const char* reuse_after; };
struct fixed_bindings : std::vector<std::pair<std::string, long long>> {
  fixed_bindings() {}
  fixed_bindings(std::initializer_list<std::pair<const char*, long long>> v) { for (const auto& x : v) push_back({x.first, x.second}); }
};
struct calls { const char* produce; const char* release = nullptr; };
struct rendezvous {
  const char* event; const char* barrier;
  rendezvous(const char* e, const char* b, all_threads_t) : event(e), barrier(b) {}
};
struct identity {
  const char* result; const char* work; const char* version; const char* dtype; const char* interpretation;
  std::vector<coord> coords;
  identity(const char* r, const char* w, const char* v, const char* d, const char* i, std::initializer_list<coord> c)
      : result(r), work(w), version(v), dtype(d), interpretation(i), coords(c) {}
  json to_json() const {
    json j = json::object(), cs = json::array();
    for (const coord& c : coords) cs.push(coord_json(c));
    j["result"] = json(result);
    j["work"] = json(work);
    j["version"] = json(version);
    j["dtype"] = json(dtype);
    j["interpretation"] = json(interpretation);
    j["coords"] = cs;
    return j;
  }
  static json coord_json(const coord& c) {
    json j = json::object();
    j["name"] = json(c.name);
    j["lo"] = json(c.lo);
    j["hi"] = json(c.hi);
    j["sort"] = json("int");
    return j;
  }
};

// one input of a map: a coordinate (every integer of [lo, hi)) or a binding (the values its PL_BINDING lists)
struct map_input {
  std::string name, sort;
  bool bound;
  std::vector<long long> points;
  json reference() const {
    json ref = json::array();
    ref.push(json(bound ? "bind" : "coord")).push(json(name));
    if (!bound || sort == "int") return ref;
    json as_int = json::array();
    as_int.push(json("toint")).push(ref);
    return as_int;
  }
};
inline map_input input_of(const coord& c) {
  map_input in{c.name, "int", false, {}};
  for (int v = c.lo; v < c.hi; ++v) in.points.push_back(v);
  return in;
}
inline map_input input_of(const bind& b) {
  map_input in{b.name, b.sort, true, {}};
  for (const auto& known : registry::get().binding_values)
    if (known.first == b.name) in.points = known.second;
  if (in.points.empty()) registry::get().fail(std::string("map input ") + b.name + " names no PL_BINDING declared before it");
  return in;
}
template <class In> struct map_argument { static int of(long long v) { return static_cast<int>(v); } };
template <> struct map_argument<bind> { static bound of(long long v) { return bound{v}; } };

// the integer-affine form of output `which` of `eval` over the inputs, as an expression; null when there is none
template <class Eval>
json fit_affine(const std::vector<map_input>& inputs, size_t which, Eval eval) {
  const size_t n = inputs.size();
  std::vector<long long> at(n), coefficient(n, 0);
  for (size_t i = 0; i < n; ++i) at[i] = inputs[i].points.empty() ? 0 : inputs[i].points[0];
  const long long origin = eval(at)[which];
  long long constant = origin;
  for (size_t i = 0; i < n; ++i) {
    if (inputs[i].points.size() < 2) continue;
    std::vector<long long> stepped = at;
    stepped[i] = inputs[i].points[1];
    const long long rise = eval(stepped)[which] - origin, run = stepped[i] - at[i];
    if (rise % run != 0) return json();
    coefficient[i] = rise / run;
    constant -= coefficient[i] * at[i];
  }
  // every point of the domain, odometer order
  std::vector<size_t> index(n, 0);
  for (bool more = true; more;) {
    long long want = constant;
    for (size_t i = 0; i < n; ++i) {
      at[i] = inputs[i].points.empty() ? 0 : inputs[i].points[index[i]];
      want += coefficient[i] * at[i];
    }
    if (eval(at)[which] != want) return json();
    more = false;
    for (size_t i = 0; i < n && !more; ++i) {
      if (inputs[i].points.empty()) continue;
      if (++index[i] < inputs[i].points.size()) more = true;
      else index[i] = 0;
    }
  }
  // terms in the order of the inputs' names, the constant last, sums nested to the left
  std::vector<size_t> order;
  for (size_t i = 0; i < n; ++i) if (coefficient[i] != 0) order.push_back(i);
  std::sort(order.begin(), order.end(), [&](size_t a, size_t b) { return inputs[a].name < inputs[b].name; });
  std::vector<json> terms;
  for (size_t i : order) {
    if (coefficient[i] == 1) { terms.push_back(inputs[i].reference()); continue; }
    json scaled = json::array();
    scaled.push(json("mulc")).push(json(coefficient[i])).push(inputs[i].reference());
    terms.push_back(scaled);
  }
  if (constant != 0 || terms.empty()) {
    json c = json::array();
    c.push(json("const")).push(json(constant));
    terms.push_back(c);
  }
  json sum = terms[0];
  for (size_t i = 1; i < terms.size(); ++i) {
    json next = json::array();
    next.push(json("add")).push(sum).push(terms[i]);
    sum = next;
  }
  return sum;
}

inline json node(const char* op, json a) { json j = json::array(); j.push(json(op)).push(std::move(a)); return j; }
inline json node(const char* op, json a, json b) { json j = json::array(); j.push(json(op)).push(std::move(a)).push(std::move(b)); return j; }
inline json fold(const char* op, const std::vector<json>& terms) {      // nested to the left
  json all = terms[0];
  for (size_t i = 1; i < terms.size(); ++i) all = node(op, all, terms[i]);
  return all;
}
inline int bit_length(unsigned long long v) { int n = 0; while (v) { ++n; v >>= 1; } return n; }

// The second family: every bit of the output is an XOR of input bits and a constant (address swizzles). The
// inputs' bits are the unknowns of one linear system over GF(2) per output bit, all output bits solved at once
// by carrying the whole output word as the right-hand side; a bit of an input that never varies gets no
// image. Printed as integer fields when no output bit mixes two input bits (x / 2^s % 2^w * 2^t), otherwise
// as masked shifts of the inputs XORed together. Inputs are taken in the order of their names.
template <class Eval>
json fit_xor_linear(const std::vector<map_input>& inputs, size_t which, Eval eval) {
  const size_t n = inputs.size();
  std::vector<size_t> order(n);
  for (size_t i = 0; i < n; ++i) order[i] = i;
  std::sort(order.begin(), order.end(), [&](size_t a, size_t b) { return inputs[a].name < inputs[b].name; });
  std::vector<int> width(n), offset(n);
  int unknowns = 1;
  for (size_t i : order) {
    long long top = 0;
    for (long long v : inputs[i].points) { if (v < 0) return json(); top = std::max(top, v); }
    width[i] = std::max(1, bit_length(static_cast<unsigned long long>(top)));
    offset[i] = unknowns;
    unknowns += width[i];
  }
  if (unknowns > 63) return json();
  std::vector<unsigned long long> row(unknowns, 0), image(unknowns, 0), solved(unknowns, 0);
  std::vector<bool> have(unknowns, false);
  std::vector<long long> at(n);
  std::vector<size_t> index(n, 0);
  int out_bits = 1;
  auto every_point = [&](auto&& visit) {
    std::fill(index.begin(), index.end(), 0);
    for (bool more = true; more;) {
      for (size_t i = 0; i < n; ++i) at[i] = inputs[i].points.empty() ? 0 : inputs[i].points[index[i]];
      if (!visit()) return false;
      more = false;
      for (size_t i = 0; i < n && !more; ++i) {
        if (inputs[i].points.empty()) continue;
        if (++index[i] < inputs[i].points.size()) more = true;
        else index[i] = 0;
      }
    }
    return true;
  };
  auto unknowns_of = [&]() {
    unsigned long long bits = 1;
    for (size_t i = 0; i < n; ++i) bits |= static_cast<unsigned long long>(at[i]) << offset[i];
    return bits;
  };
  // elimination, pivot on the lowest unknown of a row
  const bool consistent = every_point([&]() {
    const long long value = eval(at)[which];
    if (value < 0) return false;
    out_bits = std::max(out_bits, bit_length(static_cast<unsigned long long>(value)));
    unsigned long long bits = unknowns_of(), rhs = static_cast<unsigned long long>(value);
    while (bits) {
      const int pivot = bit_length(bits & (~bits + 1)) - 1;
      if (!have[pivot]) { have[pivot] = true; row[pivot] = bits; image[pivot] = rhs; break; }
      bits ^= row[pivot];
      rhs ^= image[pivot];
    }
    return bits != 0 || rhs == 0;
  });
  if (!consistent) return json();
  for (int pivot = unknowns - 1; pivot >= 0; --pivot) {
    if (!have[pivot]) continue;
    unsigned long long rhs = image[pivot];
    for (int other = pivot + 1; other < unknowns; ++other)
      if ((row[pivot] >> other) & 1) rhs ^= solved[other];
    solved[pivot] = rhs;
  }
  // integer fields: possible when every output bit copies at most one input bit
  struct origin { size_t input; int bit; };
  std::map<int, origin> source;
  bool mixing = false;
  for (size_t i : order)
    for (int b = 0; b < width[i] && !mixing; ++b)
      for (int t = 0; t < 64; ++t)
        if ((solved[offset[i] + b] >> t) & 1) {
          if (source.count(t)) { mixing = true; break; }
          source[t] = origin{i, b};
        }
  const unsigned long long constant = solved[0];
  if (!mixing) {
    std::vector<json> terms;
    int end = 0;
    for (const auto& entry : source) {
      const int target = entry.first;
      if (target < end) continue;
      const origin from = entry.second;
      const bool inverted = (constant >> target) & 1;
      int run = 1;
      for (auto next = source.find(target + run); next != source.end(); next = source.find(target + run)) {
        if (next->second.input != from.input || next->second.bit != from.bit + run || (((constant >> (target + run)) & 1) != 0) != inverted) break;
        ++run;
      }
      end = target + run;
      json term = inputs[from.input].reference();
      if (from.bit) term = node("divc", term, json(1LL << from.bit));
      if (from.bit + run < width[from.input]) term = node("modc", term, json(1LL << run));
      const long long scale = inverted ? -(1LL << target) : (1LL << target);      // c XOR x = c - x on a copied bit
      if (scale != 1) term = node("mulc", json(scale), term);
      terms.push_back(term);
    }
    if (constant != 0 || terms.empty()) terms.push_back(node("const", json(static_cast<long long>(constant))));
    return fold("add", terms);
  }
  int word = std::max(1, out_bits);
  for (size_t i = 0; i < n; ++i) word = std::max(word, width[i]);
  auto cbits = [word](unsigned long long v) { json j = json::array(); j.push(json("cbits")).push(json(word)).push(json(static_cast<long long>(v))); return j; };
  std::vector<json> terms;
  if (constant) terms.push_back(cbits(constant));
  for (size_t i : order) {
    std::map<int, unsigned long long> by_shift;        // shift -> the input bits that move by it
    for (int b = 0; b < width[i]; ++b)
      for (int t = 0; t < 64; ++t)
        if ((solved[offset[i] + b] >> t) & 1) by_shift[t - b] |= 1ULL << b;
    json as_bits = json::array();
    as_bits.push(json("tobits")).push(json(word)).push(inputs[i].reference());
    for (const auto& moved : by_shift) {
      json term = node("band", as_bits, cbits(moved.second));
      if (moved.first != 0) term = node(moved.first > 0 ? "shlc" : "shrc", term, json(moved.first > 0 ? moved.first : -moved.first));
      terms.push_back(term);
    }
  }
  if (terms.empty()) return node("const", json(0));
  return node("toint", fold("bxor", terms));
}

// a map's output as an expression: integer-affine if it is, else XOR-linear; null when it is neither
template <class Eval>
json fit_map(const std::vector<map_input>& inputs, size_t which, Eval eval) {
  json e = fit_affine(inputs, which, eval);
  return e.is_null() ? fit_xor_linear(inputs, which, eval) : e;
}

template <class Fn, class... In, size_t... I>
std::vector<long long> call_map(const Fn& fn, const std::vector<long long>& at, std::index_sequence<I...>) {
  const auto out = fn(map_argument<In>::of(at[I])...);
  return std::vector<long long>(out.begin(), out.end());
}

// pl::placement{space, units, {component names}, map, inputs...}: where an export keeps element (coords...)
struct placement {
  json record;
  template <class Fn, class... In>
  placement(const char* space, const char* units, std::initializer_list<const char*> components, Fn fn, In... in) {
    const std::vector<map_input> inputs = {input_of(in)...};
    auto eval = [&fn](const std::vector<long long>& at) { return call_map<Fn, In...>(fn, at, std::index_sequence_for<In...>{}); };
    json parts = json::object();
    size_t which = 0;
    for (const char* name : components) {
      json e = fit_map(inputs, which++, eval);
      if (e.is_null()) registry::get().fail(std::string("placement component ") + name + " is neither integer-affine nor XOR-linear in its inputs");
      parts[name] = e;
    }
    record = json::object();
    record["space"] = json(space);
    record["units"] = json(units);
    record["components"] = parts;
    record["guard"] = json();
  }
};

// pl::demand_positions{coords..., map}: thread `participant` wants element (identity coords...) at `position`
// of its destination; the map returns {identity coordinates in their declared order, participant, position}
struct demand_positions {
  std::vector<coord> domain;
  std::function<std::vector<long long>(const std::vector<long long>&)> eval;
  template <class... A>
  demand_positions(A... a) { split(std::make_tuple(a...), std::make_index_sequence<sizeof...(A) - 1>{}); }
  template <class Tuple, size_t... I>
  void split(const Tuple& t, std::index_sequence<I...>) {
    domain = {std::get<I>(t)...};
    auto fn = std::get<sizeof...(I)>(t);
    eval = [fn](const std::vector<long long>& at) {
      const auto out = fn(static_cast<int>(at[I])...);
      return std::vector<long long>(out.begin(), out.end());
    };
  }
  json to_json(const identity& id, const std::string& what) const {
    std::vector<map_input> inputs;
    json dom = json::array();
    for (const coord& c : domain) { inputs.push_back(input_of(c)); dom.push(identity::coord_json(c)); }
    auto fitted = [&](size_t which, const std::string& name) {
      json e = fit_map(inputs, which, eval);
      if (e.is_null()) registry::get().fail("demand of " + what + ": " + name + " is neither integer-affine nor XOR-linear in its inputs");
      return e;
    };
    json d = json::object(), coords = json::object();
    d["kind"] = json("positions");
    d["domain"] = dom;
    d["guard"] = json();
    const size_t k = id.coords.size();
    for (size_t i = 0; i < k; ++i) coords[id.coords[i].name] = fitted(i, id.coords[i].name);
    d["participant"] = fitted(k, "participant");
    d["position"] = fitted(k + 1, "position");
    d["identity_coords"] = coords;
    return d;
  }
};

struct reg_binding {     // PL_BINDING(name, sort, pl::values{...}, owner, units, observation scope, lifetime)
  reg_binding(const char* name, const char* sort, const values& domain, const char* owner, const char* units,
              const char* observed_at, const char* lifetime) {
    json dom = json::object(), vs = json::array();
    for (long long v : domain.items) vs.push(json(v));
    dom["name"] = json(domain.name);
    dom["sort"] = json(domain.sort);
    dom["values"] = vs;
    json b = json::object();
    b["name"] = json(name);
    b["sort"] = json(sort);
    b["domain"] = dom;
    b["owner"] = json(owner);
    b["units"] = json(units);
    b["observation_scope"] = json(observed_at);
    b["lifetime"] = json(lifetime);
    registry::get().tensor_bindings.push(b);
    registry::get().binding_values.push_back({name, domain.items});
  }
};

struct reg_site {        // PL_SITE(name, role, pl::all_threads, invocation, guarantees, observed events)
  reg_site(const char* name, const char* role, all_threads_t, const char* invocation, const guarantees& promised, const strings& observes) {
    json s = json::object();
    s["name"] = json(name);
    s["role"] = json(role);
    s["invocation"] = json(invocation);
    s["guarantees"] = promised.to_json();
    s["observes"] = observes.to_json();
    s["participants"] = json();          // every thread of the role: filled in when the roles are known
    registry::get().tensor_sites.push(s);
  }
};

struct reg_export_tensor {
  reg_export_tensor(const char* name, const identity& id, const placement& where, const strings& read_capabilities,
                    const readiness& ready, const fixed_bindings& fixed, lends backing, const ::pl::calls& through) {
    json e = json::object(), places = json::array(), rd = json::object(), fx = json::object(), cs = json::object();
    places.push(where.record);
    rd["after"] = json(ready.after);
    rd["reuse_after"] = json(ready.reuse_after);
    for (const auto& kv : fixed) fx[kv.first] = json(kv.second);
    cs["produce"] = json(through.produce);
    cs["release"] = through.release ? json(through.release) : json();
    e["name"] = json(name);
    e["identity"] = id.to_json();
    e["placements"] = places;
    e["read_capabilities"] = read_capabilities.to_json();
    e["readiness"] = rd;
    e["fixed_bindings"] = fx;
    e["backing"] = lends_json(backing);
    e["calls"] = cs;
    registry::get().tensor_exports.push(e);
  }
};

template <class F> struct argument_types;
template <class R, class... A>
struct argument_types<R(A...)> {
  static std::vector<std::string> get() { return {type_name<A>::get()...}; }
};

struct reg_import_tensor {
  // `fn` is the adapter the link generates for this import; <fn>_ready and <fn>_done are its two events
  reg_import_tensor(const char* name, const char* fn, const std::string& sig, const std::vector<std::string>& ctypes,
                    const identity& id, args meanings, const demand_positions& demand, const strings& sites,
                    const char* completion, lends lent, std::initializer_list<rendezvous> meets) {
    const size_t paren = sig.find('(');
    json callable = json::object(), events = json::object(), params = json::array();
    callable["symbol"] = json(fn);
    callable["declaration"] = json("extern \"C\" __device__ " + sig.substr(0, paren) + " " + fn + sig.substr(paren) + ";");
    events["ready"] = json(std::string(fn) + "_ready");
    events["done"] = json(std::string(fn) + "_done");
    callable["events"] = events;
    size_t k = 0;
    for (const arg& a : meanings) {
      json prm = json::object();
      prm["name"] = json(a.name);
      prm["meaning"] = json(a.meaning);
      prm["ctype"] = json(k < ctypes.size() ? ctypes[k] : std::string());
      params.push(prm);
      ++k;
    }
    if (k != ctypes.size()) registry::get().fail(std::string("import ") + name + ": pl::args names " + std::to_string(k) + " of the adapter's " + std::to_string(ctypes.size()) + " parameters");
    callable["params"] = params;
    json ms = json::array();
    for (const rendezvous& m : meets) {
      json one = json::object();
      one["event"] = json(m.event);
      one["barrier"] = json(m.barrier);
      one["cohort"] = json();            // every thread of the site's role
      ms.push(one);
    }
    json demands = json::array();
    demands.push(demand.to_json(id, name));
    json imp = json::object();
    imp["name"] = json(name);
    imp["callable"] = callable;
    imp["identity"] = id.to_json();
    imp["demands"] = demands;
    imp["sites"] = sites.to_json();
    imp["completion"] = json(completion);
    imp["lends"] = lends_json(lent);
    imp["rendezvous"] = ms;
    registry::get().tensor_imports.push(imp);
  }
};

// the entry signature every role has (docs/reference/annotations.md "Parameters and types")
template <class F>
constexpr bool is_role_entry = std::is_same<F, void(const void*, unsigned)>::value;

}  // namespace pl

#define PL_CAT2(a, b) a##b
#define PL_CAT(a, b) PL_CAT2(a, b)
#define PL_REG(type) static ::pl::type PL_CAT(pl_reg_, __COUNTER__)

#define PL_MEMBER(T, m) ::pl::member{#m, offsetof(T, m), sizeof(((T*)nullptr)->m)}
#define PL_FE_1(T, a) PL_MEMBER(T, a)
#define PL_FE_2(T, a, ...) PL_MEMBER(T, a), PL_FE_1(T, __VA_ARGS__)
#define PL_FE_3(T, a, ...) PL_MEMBER(T, a), PL_FE_2(T, __VA_ARGS__)
#define PL_FE_4(T, a, ...) PL_MEMBER(T, a), PL_FE_3(T, __VA_ARGS__)
#define PL_FE_5(T, a, ...) PL_MEMBER(T, a), PL_FE_4(T, __VA_ARGS__)
#define PL_FE_6(T, a, ...) PL_MEMBER(T, a), PL_FE_5(T, __VA_ARGS__)
#define PL_FE_7(T, a, ...) PL_MEMBER(T, a), PL_FE_6(T, __VA_ARGS__)
#define PL_FE_8(T, a, ...) PL_MEMBER(T, a), PL_FE_7(T, __VA_ARGS__)
#define PL_FE_9(T, a, ...) PL_MEMBER(T, a), PL_FE_8(T, __VA_ARGS__)
#define PL_FE_10(T, a, ...) PL_MEMBER(T, a), PL_FE_9(T, __VA_ARGS__)
#define PL_FE_11(T, a, ...) PL_MEMBER(T, a), PL_FE_10(T, __VA_ARGS__)
#define PL_FE_12(T, a, ...) PL_MEMBER(T, a), PL_FE_11(T, __VA_ARGS__)
#define PL_FE_13(T, a, ...) PL_MEMBER(T, a), PL_FE_12(T, __VA_ARGS__)
#define PL_FE_14(T, a, ...) PL_MEMBER(T, a), PL_FE_13(T, __VA_ARGS__)
#define PL_FE_15(T, a, ...) PL_MEMBER(T, a), PL_FE_14(T, __VA_ARGS__)
#define PL_FE_16(T, a, ...) PL_MEMBER(T, a), PL_FE_15(T, __VA_ARGS__)
#define PL_FE_PICK(_1, _2, _3, _4, _5, _6, _7, _8, _9, _10, _11, _12, _13, _14, _15, _16, name, ...) name
#define PL_FOR_EACH_MEMBER(T, ...)                                                                                   \
  PL_FE_PICK(__VA_ARGS__, PL_FE_16, PL_FE_15, PL_FE_14, PL_FE_13, PL_FE_12, PL_FE_11, PL_FE_10, PL_FE_9, PL_FE_8, \
             PL_FE_7, PL_FE_6, PL_FE_5, PL_FE_4, PL_FE_3, PL_FE_2, PL_FE_1)(T, __VA_ARGS__)

#define PL_STAGE(id, version) PL_REG(reg_stage)(id, version)
#define PL_PARAMS(T, ...)                                                                                      \
  static_assert(std::is_standard_layout<T>::value && std::is_trivially_copyable<T>::value,                    \
                "PL_PARAMS: a standard-layout, trivially copyable type");                                     \
  PL_REG(reg_params)(::pl::qualified_name<T>(#T).c_str(), sizeof(T), alignof(T), false, {PL_FOR_EACH_MEMBER(T, __VA_ARGS__)})
#define PL_PARAMS_OPAQUE(T) PL_REG(reg_params)(::pl::qualified_name<T>(#T).c_str(), sizeof(T), alignof(T), true, {})
#define PL_DESCRIPTOR(T) PL_REG(reg_descriptor)(sizeof(T), alignof(T))
#define PL_NO_PARAMS() PL_REG(reg_params)("void", 0, 1, false, {})
#define PL_ROLE(name, fn, warps)                                                                  \
  static_assert(::pl::is_role_entry<decltype(fn)>, "PL_ROLE: void(const void* params, unsigned variant)"); \
  PL_REG(reg_role)(#name, #fn, warps)
#define PL_EXPORT(name, fn) PL_REG(reg_export)(#name, #fn)
// PL_TYPE(T): a struct that call channels pass by pointer; the generated trampoline forward-declares it
// PL_TYPE(T, members...): the same with the members restated, checked against T's layout; declarations that
// name T then carry its definition, and a consumer needs no header of the provider's
#define PL_TYPE(T, ...) \
  namespace pl { template <> struct type_name<T> { \
    static std::string get() { return sizeof(#__VA_ARGS__) == 1 ? "struct " #T : #T; } }; } \
  struct PL_CAT(pl_type_shadow_, __LINE__) { __VA_ARGS__ }; \
  static_assert(sizeof(#__VA_ARGS__) == 1 || (sizeof(PL_CAT(pl_type_shadow_, __LINE__)) == sizeof(T) && \
                alignof(PL_CAT(pl_type_shadow_, __LINE__)) == alignof(T)), "PL_TYPE members do not restate the layout of " #T); \
  static ::pl::reg_type_if PL_CAT(pl_reg_, __COUNTER__)(#T, #__VA_ARGS__)
// PL_CALL(channel, trampoline, pl::produce, "caller_role"[, "export_name"]) at the call site;
// PL_CALL(channel, implementation, pl::consume, "export_name") beside the provided function
#define PL_CALL(channel, fn, direction, ...) \
  PL_REG(reg_call)(#channel, #fn, ::pl::signature<decltype(fn)>::get(), direction, __VA_ARGS__)
#define PL_BINDING(...) PL_REG(reg_binding)(__VA_ARGS__)
#define PL_SITE(name, ...) PL_REG(reg_site)(#name, __VA_ARGS__)
#define PL_EXPORT_TENSOR(name, ...) PL_REG(reg_export_tensor)(#name, __VA_ARGS__)
#define PL_IMPORT_TENSOR(name, fn, ...) \
  PL_REG(reg_import_tensor)(#name, #fn, ::pl::signature<decltype(fn)>::get(), ::pl::argument_types<decltype(fn)>::get(), __VA_ARGS__)
#define PL_ENDPOINT(name, ...) PL_REG(reg_endpoint){#name, __VA_ARGS__}
#define PL_CLAIM(a, b, ...) PL_REG(reg_claim_any)(#a, #b, __VA_ARGS__)
// six arguments: (domain, handle, extent, align, key, value), this header's own form; one: a pl::claim builder
#define PL_CLAIM_EX6(domain, handle, extent, align, key, value) \
  PL_REG(reg_claim)(#domain, #handle, extent, align, key, ::pl::json(value))
#define PL_CLAIM_EX1(builder) PL_REG(reg_claim_any)(builder)
#define PL_CLAIM_EX_PICK(a1, a2, a3, a4, a5, a6, which, ...) which
#define PL_CLAIM_EX(...) PL_CLAIM_EX_PICK(__VA_ARGS__, PL_CLAIM_EX6, x, x, x, x, PL_CLAIM_EX1, x)(__VA_ARGS__)
// PL_CLAIM_SMEM("handle", T[, lifetime]): shared memory sized and aligned as T
#define PL_CLAIM_SMEM(handle, T, ...) \
  PL_REG(reg_claim_any)(::pl::claim(::pl::reg_claim_any::bare(#handle).c_str(), "smem").extent(sizeof(T)).align(alignof(T)).typed().lifetime(__VA_ARGS__))
#define PL_CLAIM_WARPS(handle, role, warps, align) PL_REG(reg_warps)(#handle, #role, warps, align)
#define PL_CLAIM_REGS(handle, group, ...) PL_REG(reg_regs)(handle, group, __VA_ARGS__)
#define PL_TOPOLOGY(...) PL_REG(reg_topology){__VA_ARGS__}   // braces: no vexing parse of pl::topology()
#define PL_VARIANT(index, ...) PL_REG(reg_variant)(index, __VA_ARGS__)
#define PL_VARIANT_ENTRY(index, ...) PL_REG(reg_variant)(index, #__VA_ARGS__, __VA_ARGS__)
#define PL_HINT(key, value) PL_REG(reg_hint)(key, ::pl::json(value))

#ifndef PIPELINK_EMIT_NO_MAIN
int main() { return ::pl::emit_main(); }
#endif

#endif  // PIPELINK_EMIT
