// Registries of part kinds.  A part is looked up by (role, kind) when a model is built from its plan.
//
// Roles: "norm", "position", "mixer", "feed_forward", "arrangement", "embedding", "head".  Registering a new kind needs no
// change to this library: call register_part(role, kind, factory) (register_arrangement for a wiring) and name the kind in
// a PartSpec.  Error words that a part's kernels may raise are registered the same way.
#include <algorithm>
#include <mutex>

#include "velomind_b200/kernels.h"
#include "velomind_b200/velomind.h"

namespace vmb {

namespace {
const char* const kRoles[] = {"norm", "position", "mixer", "feed_forward", "arrangement", "embedding", "head"};

struct Registry {
    std::mutex lock;
    std::map<std::pair<std::string, std::string>, PartFactory> parts;
    std::map<std::string, ArrangementFactory> arrangements;
    std::map<int, std::string> error_words;
};
Registry& registry() {
    static Registry r;
    return r;
}

void check_role(const std::string& role) {
    for (const char* r : kRoles)
        if (role == r) return;
    std::string all;
    for (const char* r : kRoles) all += (all.empty() ? "" : ", ") + std::string(r);
    throw ConfigError(format("unknown role '%s'; roles: %s", role.c_str(), all.c_str()));
}

std::string joined(const std::vector<std::string>& v) {
    if (v.empty()) return "(none)";
    std::string s;
    for (size_t i = 0; i < v.size(); ++i) s += (i ? ", " : "") + v[i];
    return s;
}
}  // namespace

void register_part(const std::string& role, const std::string& kind, PartFactory factory) {
    check_role(role);
    if (role == "arrangement") throw ConfigError("an arrangement is built from a layer's parts: use register_arrangement");
    Registry& r = registry();
    std::lock_guard<std::mutex> g(r.lock);
    r.parts[{role, kind}] = std::move(factory);         // re-registering a kind replaces it
}

void register_arrangement(const std::string& kind, ArrangementFactory factory) {
    Registry& r = registry();
    std::lock_guard<std::mutex> g(r.lock);
    r.arrangements[kind] = std::move(factory);
}

void unregister_part(const std::string& role, const std::string& kind) {
    Registry& r = registry();
    std::lock_guard<std::mutex> g(r.lock);
    if (role == "arrangement") r.arrangements.erase(kind);
    else r.parts.erase({role, kind});
}

std::vector<std::string> registered_parts(const std::string& role) {
    Registry& r = registry();
    std::lock_guard<std::mutex> g(r.lock);
    std::vector<std::string> out;
    if (role == "arrangement")
        for (const auto& kv : r.arrangements) out.push_back(kv.first);
    else
        for (const auto& kv : r.parts)
            if (kv.first.first == role) out.push_back(kv.first.second);
    return out;
}

std::shared_ptr<Part> build_part(const std::string& role, const PartSpec& spec) {
    PartFactory factory;
    {
        Registry& r = registry();
        std::lock_guard<std::mutex> g(r.lock);
        auto it = r.parts.find({role, spec.kind});
        if (it != r.parts.end()) factory = it->second;
    }
    if (!factory)
        throw ConfigError(format("no %s of kind '%s' is registered; registered: %s", role.c_str(), spec.kind.c_str(), joined(registered_parts(role)).c_str()));
    return factory(spec.args);
}

std::shared_ptr<Arrangement> build_arrangement(const std::string& kind, const json::Value& args, const BlockParts& parts) {
    ArrangementFactory factory;
    {
        Registry& r = registry();
        std::lock_guard<std::mutex> g(r.lock);
        auto it = r.arrangements.find(kind);
        if (it != r.arrangements.end()) factory = it->second;
    }
    if (!factory)
        throw ConfigError(format("no arrangement of kind '%s' is registered; registered: %s", kind.c_str(), joined(registered_parts("arrangement")).c_str()));
    return factory(args, parts);
}

PartSpec part_spec_from_json(const json::Value& v, const std::string& what) {
    const json::Value* kind = v.find("kind");
    if (!v.is_object() || !kind || !kind->is_string()) throw ConfigError(format("%s: a part is {\"kind\": name, \"args\": {...}}", what.c_str()));
    PartSpec s;
    s.kind = kind->as_string();
    if (const json::Value* a = v.find("args")) s.args = *a;
    return s;
}

void register_error_word(int code, const std::string& meaning) {
    Registry& r = registry();
    std::lock_guard<std::mutex> g(r.lock);
    r.error_words[code] = meaning;
}

std::string error_word_meaning(int code) {
    Registry& r = registry();
    std::lock_guard<std::mutex> g(r.lock);
    auto it = r.error_words.find(code);
    return it == r.error_words.end() ? format("code %d", code) : it->second;
}

namespace {
// the words of this library's own kernels (kernels.h)
struct OwnErrorWords {
    OwnErrorWords() {
        register_error_word(VM_ERRWORD_TOKEN_ID, "a token id outside the vocabulary");
        register_error_word(VM_ERRWORD_CACHE_WRITE, "a cache write without a page");
        register_error_word(VM_ERRWORD_CACHE_READ, "a cache read without a page");
        register_error_word(VM_ERRWORD_BARRIER_WAIT, "a tensor-core kernel gave up waiting on a barrier");
    }
} own_error_words;
}  // namespace

}  // namespace vmb
