// Minimal msgpack codec (header only).
//
// The partitioning state files (deployment, profile DB, multi-level partition
// results, allocation solutions, DP cache) keep the layout the reference
// produces with msgpack-c's MSGPACK_DEFINE: every struct is a positional
// array, enums are integers, shared_ptr<T> is nil-or-T, unordered_map is a map,
// vector / unordered_set are arrays, pair is a 2-array
// (reference: src/Common.h:388-432, src/graph/DeploymentSerializer.h:11-26).
// msgpack-c itself is not available here, so this file implements the wire
// format directly on a small variant type.
#pragma once
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace rannc {
namespace mp {

struct Value;
using Array = std::vector<Value>;
using MapItems = std::vector<std::pair<Value, Value>>;

struct Value {
    enum Kind { NIL, BOOL, INT, UINT, FLOAT, STR, BIN, ARRAY, MAP } kind = NIL;
    bool b = false;
    int64_t i = 0;
    uint64_t u = 0;
    double f = 0;
    std::string s;  // STR and BIN payload
    std::shared_ptr<Array> arr;
    std::shared_ptr<MapItems> map;

    Value() = default;
    static Value nil() { return Value(); }
    static Value boolean(bool v) { Value x; x.kind = BOOL; x.b = v; return x; }
    static Value integer(int64_t v) {
        Value x;
        if (v >= 0) { x.kind = UINT; x.u = static_cast<uint64_t>(v); } else { x.kind = INT; x.i = v; }
        return x;
    }
    static Value uinteger(uint64_t v) { Value x; x.kind = UINT; x.u = v; return x; }
    static Value real(double v) { Value x; x.kind = FLOAT; x.f = v; return x; }
    static Value str(std::string v) { Value x; x.kind = STR; x.s = std::move(v); return x; }
    static Value bin(std::string v) { Value x; x.kind = BIN; x.s = std::move(v); return x; }
    static Value array(Array v = {}) { Value x; x.kind = ARRAY; x.arr = std::make_shared<Array>(std::move(v)); return x; }
    static Value mapping(MapItems v = {}) { Value x; x.kind = MAP; x.map = std::make_shared<MapItems>(std::move(v)); return x; }

    bool is_nil() const { return kind == NIL; }
    bool as_bool() const {
        if (kind == BOOL) return b;
        if (kind == UINT) return u != 0;
        if (kind == INT) return i != 0;
        throw std::runtime_error("msgpack: expected bool");
    }
    int64_t as_int() const {
        if (kind == INT) return i;
        if (kind == UINT) return static_cast<int64_t>(u);
        if (kind == BOOL) return b ? 1 : 0;
        if (kind == FLOAT) return static_cast<int64_t>(f);
        throw std::runtime_error("msgpack: expected integer");
    }
    uint64_t as_uint() const {
        if (kind == UINT) return u;
        if (kind == INT) return static_cast<uint64_t>(i);
        throw std::runtime_error("msgpack: expected unsigned integer");
    }
    double as_double() const {
        if (kind == FLOAT) return f;
        if (kind == INT) return static_cast<double>(i);
        if (kind == UINT) return static_cast<double>(u);
        throw std::runtime_error("msgpack: expected number");
    }
    const std::string& as_str() const {
        if (kind == STR || kind == BIN) return s;
        throw std::runtime_error("msgpack: expected string");
    }
    const Array& as_array() const {
        if (kind != ARRAY) throw std::runtime_error("msgpack: expected array");
        return *arr;
    }
    Array& as_array() {
        if (kind != ARRAY) throw std::runtime_error("msgpack: expected array");
        return *arr;
    }
    const MapItems& as_map() const {
        if (kind != MAP) throw std::runtime_error("msgpack: expected map");
        return *map;
    }
    const Value& at(size_t idx) const {
        const Array& a = as_array();
        if (idx >= a.size()) throw std::runtime_error("msgpack: array index out of range");
        return a[idx];
    }
};

// ------------------------------------------------------------------ encoder
class Packer {
public:
    std::string out;
    void pack(const Value& v) {
        switch (v.kind) {
            case Value::NIL: put8(0xc0); break;
            case Value::BOOL: put8(v.b ? 0xc3 : 0xc2); break;
            case Value::UINT: pack_uint(v.u); break;
            case Value::INT: pack_int(v.i); break;
            case Value::FLOAT: {
                put8(0xcb);
                uint64_t bits;
                std::memcpy(&bits, &v.f, 8);
                put64(bits);
                break;
            }
            case Value::STR: {
                const size_t n = v.s.size();
                if (n < 32) put8(0xa0 | static_cast<uint8_t>(n));
                else if (n < 256) { put8(0xd9); put8(static_cast<uint8_t>(n)); }
                else if (n < 65536) { put8(0xda); put16(static_cast<uint16_t>(n)); }
                else { put8(0xdb); put32(static_cast<uint32_t>(n)); }
                out.append(v.s);
                break;
            }
            case Value::BIN: {
                const size_t n = v.s.size();
                if (n < 256) { put8(0xc4); put8(static_cast<uint8_t>(n)); }
                else if (n < 65536) { put8(0xc5); put16(static_cast<uint16_t>(n)); }
                else { put8(0xc6); put32(static_cast<uint32_t>(n)); }
                out.append(v.s);
                break;
            }
            case Value::ARRAY: {
                const size_t n = v.arr->size();
                if (n < 16) put8(0x90 | static_cast<uint8_t>(n));
                else if (n < 65536) { put8(0xdc); put16(static_cast<uint16_t>(n)); }
                else { put8(0xdd); put32(static_cast<uint32_t>(n)); }
                for (const auto& e : *v.arr) pack(e);
                break;
            }
            case Value::MAP: {
                const size_t n = v.map->size();
                if (n < 16) put8(0x80 | static_cast<uint8_t>(n));
                else if (n < 65536) { put8(0xde); put16(static_cast<uint16_t>(n)); }
                else { put8(0xdf); put32(static_cast<uint32_t>(n)); }
                for (const auto& kv : *v.map) { pack(kv.first); pack(kv.second); }
                break;
            }
        }
    }

private:
    void put8(uint8_t x) { out.push_back(static_cast<char>(x)); }
    void put16(uint16_t x) { put8(x >> 8); put8(x & 0xff); }
    void put32(uint32_t x) { put16(x >> 16); put16(x & 0xffff); }
    void put64(uint64_t x) { put32(static_cast<uint32_t>(x >> 32)); put32(static_cast<uint32_t>(x)); }
    void pack_uint(uint64_t u) {
        if (u < 128) put8(static_cast<uint8_t>(u));
        else if (u < 256) { put8(0xcc); put8(static_cast<uint8_t>(u)); }
        else if (u < 65536) { put8(0xcd); put16(static_cast<uint16_t>(u)); }
        else if (u <= 0xffffffffull) { put8(0xce); put32(static_cast<uint32_t>(u)); }
        else { put8(0xcf); put64(u); }
    }
    void pack_int(int64_t i) {
        if (i >= 0) { pack_uint(static_cast<uint64_t>(i)); return; }
        if (i >= -32) put8(static_cast<uint8_t>(i));
        else if (i >= -128) { put8(0xd0); put8(static_cast<uint8_t>(i)); }
        else if (i >= -32768) { put8(0xd1); put16(static_cast<uint16_t>(i)); }
        else if (i >= -2147483648ll) { put8(0xd2); put32(static_cast<uint32_t>(i)); }
        else { put8(0xd3); put64(static_cast<uint64_t>(i)); }
    }
};

inline std::string pack(const Value& v) {
    Packer p;
    p.pack(v);
    return std::move(p.out);
}

// ------------------------------------------------------------------ decoder
class Unpacker {
public:
    Unpacker(const char* data, size_t size) : p_(reinterpret_cast<const uint8_t*>(data)), end_(p_ + size) {}
    Value unpack() {
        const uint8_t t = get8();
        if (t < 0x80) return Value::uinteger(t);
        if (t >= 0xe0) return Value::integer(static_cast<int8_t>(t));
        if ((t & 0xf0) == 0x80) return read_map(t & 0x0f);
        if ((t & 0xf0) == 0x90) return read_array(t & 0x0f);
        if ((t & 0xe0) == 0xa0) return Value::str(read_bytes(t & 0x1f));
        switch (t) {
            case 0xc0: return Value::nil();
            case 0xc2: return Value::boolean(false);
            case 0xc3: return Value::boolean(true);
            case 0xc4: return Value::bin(read_bytes(get8()));
            case 0xc5: return Value::bin(read_bytes(get16()));
            case 0xc6: return Value::bin(read_bytes(get32()));
            case 0xca: { uint32_t b = get32(); float f; std::memcpy(&f, &b, 4); return Value::real(f); }
            case 0xcb: { uint64_t b = get64(); double f; std::memcpy(&f, &b, 8); return Value::real(f); }
            case 0xcc: return Value::uinteger(get8());
            case 0xcd: return Value::uinteger(get16());
            case 0xce: return Value::uinteger(get32());
            case 0xcf: return Value::uinteger(get64());
            case 0xd0: return Value::integer(static_cast<int8_t>(get8()));
            case 0xd1: return Value::integer(static_cast<int16_t>(get16()));
            case 0xd2: return Value::integer(static_cast<int32_t>(get32()));
            case 0xd3: return Value::integer(static_cast<int64_t>(get64()));
            case 0xd9: return Value::str(read_bytes(get8()));
            case 0xda: return Value::str(read_bytes(get16()));
            case 0xdb: return Value::str(read_bytes(get32()));
            case 0xdc: return read_array(get16());
            case 0xdd: return read_array(get32());
            case 0xde: return read_map(get16());
            case 0xdf: return read_map(get32());
            default: throw std::runtime_error("msgpack: unsupported type byte");
        }
    }
    bool done() const { return p_ >= end_; }

private:
    const uint8_t* p_;
    const uint8_t* end_;
    void need(size_t n) { if (static_cast<size_t>(end_ - p_) < n) throw std::runtime_error("msgpack: truncated input"); }
    uint8_t get8() { need(1); return *p_++; }
    uint16_t get16() { need(2); uint16_t v = (uint16_t(p_[0]) << 8) | p_[1]; p_ += 2; return v; }
    uint32_t get32() { uint32_t hi = get16(); return (hi << 16) | get16(); }
    uint64_t get64() { uint64_t hi = get32(); return (hi << 32) | get32(); }
    std::string read_bytes(size_t n) { need(n); std::string s(reinterpret_cast<const char*>(p_), n); p_ += n; return s; }
    Value read_array(size_t n) {
        Array a;
        a.reserve(n);
        for (size_t k = 0; k < n; ++k) a.push_back(unpack());
        return Value::array(std::move(a));
    }
    Value read_map(size_t n) {
        MapItems m;
        m.reserve(n);
        for (size_t k = 0; k < n; ++k) { Value key = unpack(); Value val = unpack(); m.emplace_back(std::move(key), std::move(val)); }
        return Value::mapping(std::move(m));
    }
};

inline Value unpack(const std::string& data) {
    Unpacker u(data.data(), data.size());
    return u.unpack();
}

}  // namespace mp
}  // namespace rannc
