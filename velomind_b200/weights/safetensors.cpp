// Reader and writer for the safetensors container, with no dependency.
//
// File layout: 8 bytes little-endian header length N, N bytes of JSON (`name -> {"dtype", "shape", "data_offsets":
// [begin, end]}` plus an optional `__metadata__` object), then the raw tensor bytes.  The checks follow the reference's
// reader (src/safetensors.cpp:253-377, 412-452, 508-546): header length bounds, duplicate keys, known dtype,
// shape x dtype == byte span, spans inside the file and not overlapping.
//
// Tensors keep the STORED dtype and are views into the mapped file; nothing is cast here.
#include <algorithm>
#include <cerrno>
#include <cstdio>
#include <cstring>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include "velomind_b200/velomind.h"

namespace vmb {

namespace {
constexpr long long kMaxHeaderBytes = 100ll * 1024 * 1024;   // src/safetensors.cpp:22-23 keeps a header limit too

struct MappedFile {
    void* base = nullptr;
    size_t size = 0;
    ~MappedFile() {
        if (base && size) ::munmap(base, size);
    }
};

std::string shape_text(const std::vector<long long>& s) {
    std::string out = "[";
    for (size_t i = 0; i < s.size(); ++i) out += (i ? ", " : "") + std::to_string(s[i]);
    return out + "]";
}
}  // namespace

long long HostTensor::numel() const {
    long long n = 1;
    for (long long d : shape) n *= d;
    return n;
}

std::map<std::string, TensorEntry> parse_safetensors_header(const std::string& blob, long long data_bytes) {
    json::Value root;
    try {
        root = json::parse(blob, "safetensors header", /*no_duplicate_keys=*/true);
    } catch (const Error& e) {
        const std::string what = e.what();
        if (what.find("duplicate key") != std::string::npos) throw WeightError("duplicate key in safetensors header: " + what);
        throw WeightError("malformed safetensors header: " + what);
    }
    if (!root.is_object()) throw WeightError("safetensors header is not a JSON object");
    std::map<std::string, TensorEntry> entries;
    for (const auto& member : root.as_object()) {
        const std::string& name = member.first;
        const json::Value& desc = member.second;
        if (name == "__metadata__") continue;
        if (!desc.is_object()) throw WeightError(format("tensor '%s': entry is not an object", name.c_str()));
        const json::Value* dt = desc.find("dtype");
        std::optional<DType> dtype = (dt && dt->is_string()) ? dtype_from_name(dt->as_string()) : std::nullopt;
        if (!dtype) throw WeightError(format("tensor '%s': unsupported dtype %s", name.c_str(), dt ? dt->dump().c_str() : "(none)"));
        const json::Value* shape = desc.find("shape");
        TensorEntry e;
        e.dtype = *dtype;
        bool ok = shape && shape->is_array();
        if (ok)
            for (const auto& d : shape->as_array()) {
                if (!d.is_integer() || d.as_int() < 0) { ok = false; break; }
                e.shape.push_back(d.as_int());
            }
        if (!ok) throw WeightError(format("tensor '%s': bad shape %s", name.c_str(), shape ? shape->dump().c_str() : "(none)"));
        const json::Value* offs = desc.find("data_offsets");
        ok = offs && offs->is_array() && offs->as_array().size() == 2;
        if (ok)
            for (const auto& o : offs->as_array())
                if (!o.is_integer() || o.as_int() < 0) ok = false;
        if (!ok) throw WeightError(format("tensor '%s': bad data_offsets %s", name.c_str(), offs ? offs->dump().c_str() : "(none)"));
        e.begin = offs->as_array()[0].as_int();
        e.end = offs->as_array()[1].as_int();
        long long numel = 1;
        for (long long d : e.shape) numel *= d;
        const long long want = numel * static_cast<long long>(dtype_size(e.dtype));
        if (e.end < e.begin || e.end - e.begin != want)
            throw WeightError(format("tensor '%s': shape %s of %s needs %lld bytes, data_offsets span %lld", name.c_str(),
                                     shape_text(e.shape).c_str(), dtype_name(e.dtype), want, e.end - e.begin));
        if (e.end > data_bytes)
            throw WeightError(format("tensor '%s': data_offsets end %lld beyond the payload (%lld bytes): truncated file?", name.c_str(),
                                     e.end, data_bytes));
        entries[name] = std::move(e);
    }
    std::vector<std::tuple<long long, long long, std::string>> spans;
    for (const auto& kv : entries)
        if (kv.second.end > kv.second.begin) spans.emplace_back(kv.second.begin, kv.second.end, kv.first);
    std::sort(spans.begin(), spans.end());
    for (size_t i = 1; i < spans.size(); ++i)
        if (std::get<0>(spans[i]) < std::get<1>(spans[i - 1]))
            throw WeightError(format("tensors '%s' and '%s' overlap in the payload", std::get<2>(spans[i - 1]).c_str(), std::get<2>(spans[i]).c_str()));
    return entries;
}

HostTensors load_safetensors(const std::string& path) {
    const int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0) throw WeightError(format("%s: cannot open (%s)", path.c_str(), std::strerror(errno)));
    struct stat st;
    if (::fstat(fd, &st) != 0) { ::close(fd); throw WeightError(path + ": cannot stat"); }
    const long long size = st.st_size;
    if (size < 8) { ::close(fd); throw WeightError(path + ": shorter than the 8-byte length prefix"); }
    auto mapped = std::make_shared<MappedFile>();
    mapped->base = ::mmap(nullptr, static_cast<size_t>(size), PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (mapped->base == MAP_FAILED) { mapped->base = nullptr; throw WeightError(path + ": cannot map the file"); }
    mapped->size = static_cast<size_t>(size);
    const uint8_t* bytes = static_cast<const uint8_t*>(mapped->base);
    unsigned long long n = 0;
    for (int i = 7; i >= 0; --i) n = (n << 8) | bytes[i];
    if (n == 0 || n > static_cast<unsigned long long>(kMaxHeaderBytes) || 8 + n > static_cast<unsigned long long>(size))
        throw WeightError(format("%s: header length %llu is not plausible for a file of %lld bytes", path.c_str(), n, size));
    const std::string blob(reinterpret_cast<const char*>(bytes + 8), static_cast<size_t>(n));
    std::map<std::string, TensorEntry> entries;
    try {
        entries = parse_safetensors_header(blob, size - 8 - static_cast<long long>(n));
    } catch (const WeightError& e) {
        throw WeightError(path + ": " + e.what());
    }
    const uint8_t* payload = bytes + 8 + n;
    HostTensors out;
    for (auto& kv : entries) {
        HostTensor t;
        t.dtype = kv.second.dtype;
        t.shape = kv.second.shape;
        t.data = payload + kv.second.begin;
        t.nbytes = static_cast<size_t>(kv.second.end - kv.second.begin);
        t.owner = mapped;
        out[kv.first] = std::move(t);
    }
    return out;
}

void save_safetensors(const HostTensors& tensors, const std::string& path, const std::map<std::string, std::string>& metadata) {
    json::Value header;
    header.object();
    if (!metadata.empty()) {
        json::Value md;
        for (const auto& kv : metadata) md.set(kv.first, kv.second);
        header.set("__metadata__", md);
    }
    long long off = 0;
    for (const auto& kv : tensors) {           // std::map: names sorted
        json::Value d;
        d.set("dtype", dtype_name(kv.second.dtype));
        json::Array shape;
        for (long long s : kv.second.shape) shape.emplace_back(s);
        d.set("shape", std::move(shape));
        d.set("data_offsets", json::Array{json::Value(off), json::Value(off + static_cast<long long>(kv.second.nbytes))});
        header.set(kv.first, d);
        off += static_cast<long long>(kv.second.nbytes);
    }
    std::string blob = header.dump();
    while (blob.size() % 8) blob.push_back(' ');
    const std::string tmp = path + ".tmp";
    FILE* f = std::fopen(tmp.c_str(), "wb");
    if (!f) throw WeightError(format("%s: cannot write (%s)", tmp.c_str(), std::strerror(errno)));
    uint8_t len[8];
    unsigned long long n = blob.size();
    for (int i = 0; i < 8; ++i) len[i] = static_cast<uint8_t>((n >> (8 * i)) & 0xff);
    bool ok = std::fwrite(len, 1, 8, f) == 8 && std::fwrite(blob.data(), 1, blob.size(), f) == blob.size();
    for (const auto& kv : tensors)
        if (ok && kv.second.nbytes) ok = std::fwrite(kv.second.data, 1, kv.second.nbytes, f) == kv.second.nbytes;
    ok = (std::fclose(f) == 0) && ok;
    if (!ok || std::rename(tmp.c_str(), path.c_str()) != 0) throw WeightError(path + ": write failed");
}

}  // namespace vmb
