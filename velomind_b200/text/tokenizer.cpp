// Byte-level BPE tokenizer read from a Hugging Face `tokenizer.json` (optional: generation works on token ids without it),
// and the streamer that turns a growing token list into pieces of text.
//
// Behaviour follows the reference's tokenizer (examples/smollm2/tokenizer.cpp): fields `model.vocab`, `model.merges`,
// `added_tokens` (:77-167); special ids inferred from the token text (:153-166); the GPT-2 byte <-> unicode table; a
// hand-written pre-tokenizer (contractions, runs of letters with one leading space, single digits, runs of other symbols,
// runs of whitespace; :236-368); lowest-rank-first merges (:370-429); decoding skips the begin/end/pad ids (:466-498).
// One deliberate difference: after a space, the reference glues that space to EVERY digit of a number (" 12" -> " 1", " 2"),
// which does not decode back to the input; here the space is a piece of its own and digits stand alone.
// Letters beyond ASCII: every code point from U+0080 on counts as a letter unless it lies in a block of spaces,
// punctuation or symbols listed in `is_alpha` below.
#include <fstream>
#include <sstream>

#include "velomind_b200/velomind.h"

namespace vmb {

namespace {

// ---- UTF-8
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

// One code point of `s` at `i`; `len` receives the bytes it takes.  Invalid or truncated: U+FFFD and the length of the longest
// prefix that could have begun a character (at least one byte).
unsigned next_code_point(const std::string& s, size_t i, size_t& len) {
    const unsigned char c = static_cast<unsigned char>(s[i]);
    auto cont = [&](size_t k) { return i + k < s.size() && (static_cast<unsigned char>(s[i + k]) & 0xC0) == 0x80; };
    len = 1;
    if (c < 0x80) return c;
    int need = 0;
    unsigned cp = 0;
    unsigned lo = 0x80, hi = 0xBF;           // allowed range of the first continuation byte
    if (c >= 0xC2 && c <= 0xDF) { need = 1; cp = c & 0x1F; }
    else if (c >= 0xE0 && c <= 0xEF) { need = 2; cp = c & 0x0F; if (c == 0xE0) lo = 0xA0; if (c == 0xED) hi = 0x9F; }
    else if (c >= 0xF0 && c <= 0xF4) { need = 3; cp = c & 0x07; if (c == 0xF0) lo = 0x90; if (c == 0xF4) hi = 0x8F; }
    else return 0xFFFD;
    for (int k = 1; k <= need; ++k) {
        if (!cont(static_cast<size_t>(k))) { len = static_cast<size_t>(k); return 0xFFFD; }
        const unsigned char b = static_cast<unsigned char>(s[i + static_cast<size_t>(k)]);
        if (k == 1 && (b < lo || b > hi)) { len = 1; return 0xFFFD; }
        cp = (cp << 6) | (b & 0x3F);
    }
    len = static_cast<size_t>(need) + 1;
    return cp;
}

std::vector<unsigned> code_points(const std::string& s) {
    std::vector<unsigned> out;
    for (size_t i = 0; i < s.size();) {
        size_t len;
        out.push_back(next_code_point(s, i, len));
        i += len;
    }
    return out;
}

std::string sanitized(const std::string& bytes) {       // invalid sequences become U+FFFD
    std::string out;
    for (size_t i = 0; i < bytes.size();) {
        size_t len;
        const unsigned cp = next_code_point(bytes, i, len);
        if (cp == 0xFFFD) append_utf8(0xFFFD, out);
        else out.append(bytes, i, len);
        i += len;
    }
    return out;
}

bool is_space(unsigned c) {
    return c == ' ' || (c >= 0x09 && c <= 0x0D) || (c >= 0x1C && c <= 0x1F) || c == 0x85 || c == 0xA0 || c == 0x1680 || (c >= 0x2000 && c <= 0x200A) ||
           c == 0x2028 || c == 0x2029 || c == 0x202F || c == 0x205F || c == 0x3000;
}
bool is_digit(unsigned c) { return c >= '0' && c <= '9'; }
bool is_alpha(unsigned c) {
    if (c < 0x80) return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z');
    if (is_space(c)) return false;
    if (c >= 0x80 && c <= 0xBF) return c == 0xAA || c == 0xB5 || c == 0xBA;      // Latin-1 punctuation and signs, but for three letters
    if (c == 0xD7 || c == 0xF7) return false;
    if (c >= 0x2010 && c <= 0x2BFF) return false;       // general punctuation, currency, arrows, mathematical and technical signs, shapes
    if (c >= 0x3001 && c <= 0x303F) return false;       // CJK punctuation
    if (c >= 0xFE10 && c <= 0xFE6F) return false;
    if ((c >= 0xFF01 && c <= 0xFF0F) || (c >= 0xFF1A && c <= 0xFF20) || (c >= 0xFF3B && c <= 0xFF40) || (c >= 0xFF5B && c <= 0xFF65)) return false;
    if (c >= 0x1F000 && c <= 0x1FAFF) return false;     // emoji and pictographs
    if (c == 0xFFFD) return false;
    return true;
}

// ---- the GPT-2 byte <-> unicode table
struct ByteTable {
    unsigned to_uni[256];
    std::unordered_map<unsigned, unsigned char> to_byte;
    ByteTable() {
        unsigned extra = 0;
        for (unsigned b = 0; b < 256; ++b) {
            const bool keep = (b >= '!' && b <= '~') || (b >= 0xA1 && b <= 0xAC) || (b >= 0xAE && b <= 0xFF);
            to_uni[b] = keep ? b : 256 + extra++;
            to_byte[to_uni[b]] = static_cast<unsigned char>(b);
        }
    }
};
const ByteTable& byte_table() {
    static ByteTable t;
    return t;
}

const char* const kContractions[] = {"'s", "'t", "'m", "'d", "'re", "'ve", "'ll"};

}  // namespace

std::vector<std::string> Tokenizer::pretokenize(const std::string& text) {
    const std::vector<unsigned> cps = code_points(text);
    const size_t n = cps.size();
    std::vector<std::string> pieces;
    size_t i = 0;
    auto starts_with = [&](size_t at, const char* lit) {
        for (size_t k = 0; lit[k]; ++k)
            if (at + k >= n || cps[at + k] != static_cast<unsigned char>(lit[k])) return false;
        return true;
    };
    while (i < n) {
        size_t j = i;
        const char* hit = nullptr;
        for (const char* c : kContractions)
            if (starts_with(i, c)) { hit = c; break; }
        if (hit) j = i + std::string(hit).size();
        else {
            const unsigned ch = cps[i];
            if (ch == ' ' && i + 1 < n && is_alpha(cps[i + 1])) {
                j = i + 1;
                while (j < n && is_alpha(cps[j])) ++j;
            } else if (is_alpha(ch)) {
                while (j < n && is_alpha(cps[j])) ++j;
            } else if (is_digit(ch)) {
                j = i + 1;                                   // digits stand alone
            } else if (!is_space(ch)) {
                while (j < n && !(is_space(cps[j]) || is_alpha(cps[j]) || is_digit(cps[j]))) ++j;
            } else if (ch == ' ' && i + 1 < n && is_digit(cps[i + 1])) {
                j = i + 1;                                   // the space before a number is its own piece
            } else {
                while (j < n && is_space(cps[j])) ++j;
            }
        }
        std::string raw;
        for (size_t k = i; k < j; ++k) append_utf8(cps[k], raw);
        std::string mapped;
        for (unsigned char b : raw) append_utf8(byte_table().to_uni[b], mapped);
        pieces.push_back(mapped);
        i = j;
    }
    return pieces;
}

std::shared_ptr<Tokenizer> Tokenizer::from_file(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw Error(path + ": cannot open");
    std::stringstream ss;
    ss << f.rdbuf();
    return from_json(json::parse(ss.str(), path, /*no_duplicate_keys=*/false), path);
}

std::shared_ptr<Tokenizer> Tokenizer::from_json(const json::Value& root, const std::string& where) {
    const json::Value* model = root.find("model");
    const json::Value* vocab = model ? model->find("vocab") : nullptr;
    if (!vocab || !vocab->is_object() || vocab->as_object().empty()) throw Error(where + ": no model.vocab object");
    auto tok = std::make_shared<Tokenizer>();
    int size = 0;
    for (const auto& m : vocab->as_object())
        if (m.second.is_integer()) {
            tok->token_to_id_[m.first] = static_cast<int>(m.second.as_int());
            size = std::max(size, static_cast<int>(m.second.as_int()) + 1);
        }
    if (const json::Value* merges = model->find("merges")) {
        int r = 0;
        for (const auto& m : merges->as_array()) {
            if (m.is_string()) tok->rank_.emplace(m.as_string(), r++);                       // "a b"
            else if (m.is_array() && m.as_array().size() == 2 && m.as_array()[0].is_string() && m.as_array()[1].is_string())
                tok->rank_.emplace(m.as_array()[0].as_string() + " " + m.as_array()[1].as_string(), r++);
        }
    }
    std::vector<std::pair<std::string, int>> added;
    if (const json::Value* at = root.find("added_tokens"))
        for (const auto& t : at->as_array()) {
            const json::Value *content = t.find("content"), *id = t.find("id");
            if (content && content->is_string() && id && id->is_integer()) added.emplace_back(content->as_string(), static_cast<int>(id->as_int()));
        }
    for (const auto& a : added) {
        tok->token_to_id_[a.first] = a.second;
        size = std::max(size, a.second + 1);
    }
    tok->id_to_token_.assign(static_cast<size_t>(size), "");
    for (const auto& kv : tok->token_to_id_)
        if (kv.second >= 0) tok->id_to_token_[static_cast<size_t>(kv.second)] = kv.first;
    for (const auto& a : added) {                 // special ids inferred from the token text (tokenizer.cpp:153-166)
        const std::string& t = a.first;
        if (t == "<|endoftext|>" || t == "<s>" || t == "<bos>") {
            tok->bos_id = a.second;
            if (tok->eos_id < 0) tok->eos_id = a.second;
        } else if (t == "<|im_end|>" || t == "</s>" || t == "<eos>") tok->eos_id = a.second;
        else if (t == "<pad>" || t == "<|padding|>") tok->pad_id = a.second;
        else if (t == "<unk>") tok->unk_id = a.second;
    }
    if (tok->bos_id < 0 && tok->eos_id >= 0) tok->bos_id = tok->eos_id;
    return tok;
}

std::vector<std::string> Tokenizer::bpe(const std::string& word) const {
    std::vector<std::string> symbols;
    for (size_t i = 0; i < word.size();) {
        size_t len;
        next_code_point(word, i, len);
        symbols.push_back(word.substr(i, len));
        i += len;
    }
    while (symbols.size() > 1) {
        int best = -1;
        size_t at = 0;
        for (size_t i = 0; i + 1 < symbols.size(); ++i) {
            auto it = rank_.find(symbols[i] + " " + symbols[i + 1]);
            if (it != rank_.end() && (best < 0 || it->second < best)) { best = it->second; at = i; }
        }
        if (best < 0) break;
        symbols[at] += symbols[at + 1];
        symbols.erase(symbols.begin() + static_cast<long>(at) + 1);
    }
    return symbols;
}

std::vector<int> Tokenizer::encode(const std::string& text) const {
    std::vector<int> out;
    for (const std::string& piece : pretokenize(text)) {
        auto whole = token_to_id_.find(piece);
        if (whole != token_to_id_.end()) { out.push_back(whole->second); continue; }
        for (const std::string& sym : bpe(piece)) {
            auto it = token_to_id_.find(sym);
            if (it != token_to_id_.end()) out.push_back(it->second);
            else if (unk_id >= 0) out.push_back(unk_id);
        }
    }
    return out;
}

std::string Tokenizer::decode(const std::vector<int>& ids) const {
    std::string bytes;
    for (int id : ids) {
        if (id < 0 || id >= static_cast<int>(id_to_token_.size()) || id == bos_id || id == eos_id || id == pad_id) continue;
        const std::string& t = id_to_token_[static_cast<size_t>(id)];
        for (size_t i = 0; i < t.size();) {
            size_t len;
            const unsigned cp = next_code_point(t, i, len);
            auto b = byte_table().to_byte.find(cp);
            if (b != byte_table().to_byte.end()) bytes.push_back(static_cast<char>(b->second));
            else bytes.append(t, i, len);
            i += len;
        }
    }
    return sanitized(bytes);
}

// ------------------------------------------------------------------------------------------------ TextStreamer
std::string TextStreamer::put(int token) {
    if (!tokenizer_) return format("[%d]", token);
    tokens_.push_back(token);
    const std::string text = tokenizer_->decode(tokens_);
    static const std::string kReplacement = "\xEF\xBF\xBD";
    if (text.size() >= 3 && text.compare(text.size() - 3, 3, kReplacement) == 0) return "";   // the bytes so far end inside a character: wait
    if (text.size() < emitted_) { emitted_ = text.size(); return ""; }
    std::string piece = text.substr(emitted_);
    emitted_ = text.size();
    return piece;
}

std::string TextStreamer::flush() {
    if (!tokenizer_) return "";
    const std::string text = tokenizer_->decode(tokens_);
    if (text.size() <= emitted_) return "";
    std::string piece = text.substr(emitted_);
    emitted_ = text.size();
    return piece;
}

}  // namespace vmb
