// args.h (internal) — reading a part's constructor arguments (a JSON object of sizes and constants) with errors that
// name the argument, and the helper that registers a part kind when the library is loaded.
#pragma once

#include <cmath>

#include "velomind_b200/velomind.h"

namespace vmb {

inline long long arg_int(const json::Value& args, const char* name, const char* part) {
    const json::Value* v = args.find(name);
    if (!v || !v->is_integer()) throw ConfigError(format("part '%s': argument '%s' must be an integer", part, name));
    return v->as_int();
}

inline long long arg_int_or(const json::Value& args, const char* name, long long fallback, const char* part) {
    const json::Value* v = args.find(name);
    if (!v || v->is_null()) return fallback;
    if (!v->is_integer()) throw ConfigError(format("part '%s': argument '%s' must be an integer", part, name));
    return v->as_int();
}

inline double arg_number(const json::Value& args, const char* name, const char* part) {
    const json::Value* v = args.find(name);
    if (!v || !v->is_number() || !std::isfinite(v->as_double())) throw ConfigError(format("part '%s': argument '%s' must be a number", part, name));
    return v->as_double();
}

inline double arg_number_or(const json::Value& args, const char* name, double fallback, const char* part) {
    const json::Value* v = args.find(name);
    if (!v || v->is_null()) return fallback;
    return arg_number(args, name, part);
}

inline std::string arg_string_or(const json::Value& args, const char* name, const std::string& fallback, const char* part) {
    const json::Value* v = args.find(name);
    if (!v || v->is_null()) return fallback;
    if (!v->is_string()) throw ConfigError(format("part '%s': argument '%s' must be a string", part, name));
    return v->as_string();
}

struct RegisterPart {
    RegisterPart(const char* role, const char* kind, PartFactory f) { register_part(role, kind, std::move(f)); }
};

}  // namespace vmb
