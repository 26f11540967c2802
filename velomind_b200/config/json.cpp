// A small JSON reader and writer: config.json, the safetensors header, tokenizer.json, traces, plans.
// (The reference scans config.json for substrings, examples/smollm2/config_parser.cpp:134-216, and has a second
// hand-written parser for the safetensors header, src/safetensors.cpp:60-250; here one real parser serves all.)
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "velomind_b200/velomind.h"

namespace vmb {

std::string format(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    va_list ap2;
    va_copy(ap2, ap);
    const int n = std::vsnprintf(nullptr, 0, fmt, ap);
    va_end(ap);
    std::string out(n > 0 ? static_cast<size_t>(n) : 0, '\0');
    if (n > 0) std::vsnprintf(out.data(), static_cast<size_t>(n) + 1, fmt, ap2);
    va_end(ap2);
    return out;
}

namespace json {

Value::Value(Array a) : kind_(ArrayKind), arr_(std::make_shared<Array>(std::move(a))) {}
Value::Value(Object o) : kind_(ObjectKind), obj_(std::make_shared<Object>(std::move(o))) {}

static const Array kEmptyArray;
static const Object kEmptyObject;

const Array& Value::as_array() const { return arr_ ? *arr_ : kEmptyArray; }
const Object& Value::as_object() const { return obj_ ? *obj_ : kEmptyObject; }

Array& Value::array() {
    if (kind_ != ArrayKind) { *this = Value(Array{}); }
    if (arr_.use_count() > 1) arr_ = std::make_shared<Array>(*arr_);
    return *arr_;
}

Object& Value::object() {
    if (kind_ != ObjectKind) { *this = Value(Object{}); }
    if (obj_.use_count() > 1) obj_ = std::make_shared<Object>(*obj_);
    return *obj_;
}

const Value* Value::find(const std::string& key) const {
    if (kind_ != ObjectKind) return nullptr;
    for (const auto& m : *obj_)
        if (m.first == key) return &m.second;
    return nullptr;
}

void Value::set(const std::string& key, Value v) {
    Object& o = object();
    for (auto& m : o)
        if (m.first == key) { m.second = std::move(v); return; }
    o.emplace_back(key, std::move(v));
}

bool Value::operator==(const Value& o) const {
    if (kind_ != o.kind_) return false;
    switch (kind_) {
        case Null: return true;
        case Bool: return b_ == o.b_;
        case Number: return num_ == o.num_;
        case String: return str_ == o.str_;
        case ArrayKind: return as_array() == o.as_array();
        case ObjectKind: {
            const Object &a = as_object(), &b = o.as_object();
            if (a.size() != b.size()) return false;
            for (const auto& m : a) {
                const Value* other = o.find(m.first);
                if (!other || !(*other == m.second)) return false;
            }
            return true;
        }
    }
    return false;
}

static void dump_string(const std::string& s, std::string& out) {
    out.push_back('"');
    for (unsigned char c : s) {
        switch (c) {
            case '"': out += "\\\""; break;
            case '\\': out += "\\\\"; break;
            case '\n': out += "\\n"; break;
            case '\r': out += "\\r"; break;
            case '\t': out += "\\t"; break;
            case '\b': out += "\\b"; break;
            case '\f': out += "\\f"; break;
            default:
                if (c < 0x20) out += format("\\u%04x", c);
                else out.push_back(static_cast<char>(c));
        }
    }
    out.push_back('"');
}

static void dump_value(const Value& v, int indent, int depth, std::string& out) {
    auto newline = [&](int d) {
        if (indent < 0) return;
        out.push_back('\n');
        out.append(static_cast<size_t>(indent * d), ' ');
    };
    switch (v.kind()) {
        case Value::Null: out += "null"; break;
        case Value::Bool: out += v.as_bool() ? "true" : "false"; break;
        case Value::Number:
            if (v.is_integer()) out += format("%lld", v.as_int());
            else if (!std::isfinite(v.as_double())) out += "null";
            else out += format("%.17g", v.as_double());
            break;
        case Value::String: dump_string(v.as_string(), out); break;
        case Value::ArrayKind: {
            const Array& a = v.as_array();
            out.push_back('[');
            for (size_t i = 0; i < a.size(); ++i) {
                if (i) out += indent < 0 ? ", " : ",";
                if (a[i].is_array() || a[i].is_object()) newline(depth + 1);
                dump_value(a[i], indent, depth + 1, out);
            }
            out.push_back(']');
            break;
        }
        case Value::ObjectKind: {
            const Object& o = v.as_object();
            out.push_back('{');
            for (size_t i = 0; i < o.size(); ++i) {
                if (i) out += indent < 0 ? ", " : ",";
                newline(depth + 1);
                dump_string(o[i].first, out);
                out += ": ";
                dump_value(o[i].second, indent, depth + 1, out);
            }
            if (!o.empty()) newline(depth);
            out.push_back('}');
            break;
        }
    }
}

std::string Value::dump(int indent) const {
    std::string out;
    dump_value(*this, indent, 0, out);
    return out;
}

namespace {

struct Parser {
    const std::string& s;
    const std::string& where;
    bool no_dups;
    size_t i = 0;
    int depth = 0;

    [[noreturn]] void fail(const std::string& what) const {
        throw Error(format("%s: not valid JSON: %s at byte %zu", where.c_str(), what.c_str(), i));
    }
    void skip() {
        while (i < s.size() && (s[i] == ' ' || s[i] == '\t' || s[i] == '\n' || s[i] == '\r')) ++i;
    }
    Value value() {
        skip();
        if (i >= s.size()) fail("unexpected end");
        if (++depth > 200) fail("nesting too deep");
        Value v;
        const char c = s[i];
        if (c == '{') v = object();
        else if (c == '[') v = array();
        else if (c == '"') v = Value(string());
        else if (c == 't' || c == 'f' || c == 'n') v = literal();
        else if (c == '-' || (c >= '0' && c <= '9')) v = number();
        else fail(format("unexpected character '%c'", c));
        --depth;
        return v;
    }
    Value literal() {
        if (s.compare(i, 4, "true") == 0) { i += 4; return Value(true); }
        if (s.compare(i, 5, "false") == 0) { i += 5; return Value(false); }
        if (s.compare(i, 4, "null") == 0) { i += 4; return Value(); }
        fail("unknown literal");
    }
    Value number() {
        const size_t start = i;
        bool integral = true;
        if (s[i] == '-') ++i;
        if (i >= s.size() || !(s[i] >= '0' && s[i] <= '9')) fail("bad number");
        while (i < s.size() && s[i] >= '0' && s[i] <= '9') ++i;
        if (i < s.size() && s[i] == '.') {
            integral = false;
            ++i;
            if (i >= s.size() || !(s[i] >= '0' && s[i] <= '9')) fail("bad number");
            while (i < s.size() && s[i] >= '0' && s[i] <= '9') ++i;
        }
        if (i < s.size() && (s[i] == 'e' || s[i] == 'E')) {
            integral = false;
            ++i;
            if (i < s.size() && (s[i] == '+' || s[i] == '-')) ++i;
            if (i >= s.size() || !(s[i] >= '0' && s[i] <= '9')) fail("bad number");
            while (i < s.size() && s[i] >= '0' && s[i] <= '9') ++i;
        }
        const std::string text = s.substr(start, i - start);
        if (integral && text.size() <= 18) return Value(static_cast<long long>(std::strtoll(text.c_str(), nullptr, 10)));
        const double d = std::strtod(text.c_str(), nullptr);
        // a whole number written with a fraction or exponent (1e5, 64.0) still counts as an integer where one is asked for
        if (std::isfinite(d) && std::fabs(d) < 9e15 && d == std::floor(d)) {
            Value v(static_cast<long long>(d));
            return v;
        }
        return Value(d);
    }
    void append_utf8(unsigned cp, std::string& out) {
        if (cp < 0x80) out.push_back(static_cast<char>(cp));
        else if (cp < 0x800) { out.push_back(static_cast<char>(0xC0 | (cp >> 6))); out.push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
        else if (cp < 0x10000) {
            out.push_back(static_cast<char>(0xE0 | (cp >> 12)));
            out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
            out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
        } else {
            out.push_back(static_cast<char>(0xF0 | (cp >> 18)));
            out.push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
            out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
            out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
        }
    }
    unsigned hex4() {
        if (i + 4 > s.size()) fail("bad \\u escape");
        unsigned v = 0;
        for (int k = 0; k < 4; ++k) {
            const char c = s[i++];
            v <<= 4;
            if (c >= '0' && c <= '9') v |= static_cast<unsigned>(c - '0');
            else if (c >= 'a' && c <= 'f') v |= static_cast<unsigned>(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= static_cast<unsigned>(c - 'A' + 10);
            else fail("bad \\u escape");
        }
        return v;
    }
    std::string string() {
        ++i;  // opening quote
        std::string out;
        while (true) {
            if (i >= s.size()) fail("unterminated string");
            const unsigned char c = static_cast<unsigned char>(s[i++]);
            if (c == '"') break;
            if (c < 0x20) fail("control character in string");
            if (c != '\\') { out.push_back(static_cast<char>(c)); continue; }
            if (i >= s.size()) fail("unterminated string");
            const char e = s[i++];
            switch (e) {
                case '"': out.push_back('"'); break;
                case '\\': out.push_back('\\'); break;
                case '/': out.push_back('/'); break;
                case 'b': out.push_back('\b'); break;
                case 'f': out.push_back('\f'); break;
                case 'n': out.push_back('\n'); break;
                case 'r': out.push_back('\r'); break;
                case 't': out.push_back('\t'); break;
                case 'u': {
                    unsigned cp = hex4();
                    if (cp >= 0xD800 && cp <= 0xDBFF && i + 1 < s.size() && s[i] == '\\' && s[i + 1] == 'u') {
                        i += 2;
                        const unsigned lo = hex4();
                        if (lo >= 0xDC00 && lo <= 0xDFFF) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                        else { append_utf8(0xFFFD, out); cp = lo; }
                    }
                    append_utf8(cp, out);
                    break;
                }
                default: fail("unknown escape");
            }
        }
        return out;
    }
    Value array() {
        ++i;
        Array a;
        skip();
        if (i < s.size() && s[i] == ']') { ++i; return Value(std::move(a)); }
        while (true) {
            a.push_back(value());
            skip();
            if (i >= s.size()) fail("unterminated array");
            if (s[i] == ',') { ++i; continue; }
            if (s[i] == ']') { ++i; break; }
            fail("expected ',' or ']'");
        }
        return Value(std::move(a));
    }
    Value object() {
        ++i;
        Object o;
        skip();
        if (i < s.size() && s[i] == '}') { ++i; return Value(std::move(o)); }
        while (true) {
            skip();
            if (i >= s.size() || s[i] != '"') fail("expected a key");
            std::string key = string();
            if (no_dups)
                for (const auto& m : o)
                    if (m.first == key) fail(format("duplicate key '%s'", key.c_str()));
            skip();
            if (i >= s.size() || s[i] != ':') fail("expected ':'");
            ++i;
            Value v = value();
            o.emplace_back(std::move(key), std::move(v));
            skip();
            if (i >= s.size()) fail("unterminated object");
            if (s[i] == ',') { ++i; continue; }
            if (s[i] == '}') { ++i; break; }
            fail("expected ',' or '}'");
        }
        return Value(std::move(o));
    }
};

}  // namespace

Value parse(const std::string& text, const std::string& where, bool no_duplicate_keys) {
    Parser p{text, where, no_duplicate_keys};
    Value v = p.value();
    p.skip();
    if (p.i != text.size()) p.fail("text after the value");
    return v;
}

}  // namespace json
}  // namespace vmb
