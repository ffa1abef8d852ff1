#include "dnn/tokens/vocab_loader.cuh"

#include <cstdint>
#include <fstream>
#include <sstream>
#include <stdexcept>

namespace dnn {

namespace {

// ---- a reader for the one JSON shape a vocabulary file has: a flat object of string keys and integer values ----

struct JsonCursor {
    const std::string& s;
    size_t i = 0;
    void skip_space() {
        while (i < s.size() && (s[i] == ' ' || s[i] == '\t' || s[i] == '\n' || s[i] == '\r')) ++i;
    }
    [[noreturn]] void fail(const char* what) const {
        throw std::runtime_error("Failed to parse vocabulary JSON: " + std::string(what) + " at offset " + std::to_string(i));
    }
    char peek() {
        skip_space();
        if (i >= s.size()) fail("unexpected end of input");
        return s[i];
    }
    void expect(char c) {
        if (peek() != c) fail("unexpected character");
        ++i;
    }
};

void append_utf8(std::string& out, uint32_t cp) {
    if (cp < 0x80) {
        out += char(cp);
    } else if (cp < 0x800) {
        out += char(0xC0 | (cp >> 6));
        out += char(0x80 | (cp & 0x3F));
    } else if (cp < 0x10000) {
        out += char(0xE0 | (cp >> 12));
        out += char(0x80 | ((cp >> 6) & 0x3F));
        out += char(0x80 | (cp & 0x3F));
    } else {
        out += char(0xF0 | (cp >> 18));
        out += char(0x80 | ((cp >> 12) & 0x3F));
        out += char(0x80 | ((cp >> 6) & 0x3F));
        out += char(0x80 | (cp & 0x3F));
    }
}

uint32_t hex4(JsonCursor& c) {
    if (c.i + 4 > c.s.size()) c.fail("truncated \\u escape");
    uint32_t v = 0;
    for (int k = 0; k < 4; ++k) {
        const char h = c.s[c.i++];
        v <<= 4;
        if (h >= '0' && h <= '9') v |= uint32_t(h - '0');
        else if (h >= 'a' && h <= 'f') v |= uint32_t(h - 'a' + 10);
        else if (h >= 'A' && h <= 'F') v |= uint32_t(h - 'A' + 10);
        else c.fail("bad \\u escape");
    }
    return v;
}

std::string parse_string(JsonCursor& c) {
    c.expect('"');
    std::string out;
    for (;;) {
        if (c.i >= c.s.size()) c.fail("unterminated string");
        const char ch = c.s[c.i++];
        if (ch == '"') return out;
        if (ch != '\\') {
            out += ch;
            continue;
        }
        if (c.i >= c.s.size()) c.fail("unterminated escape");
        const char e = c.s[c.i++];
        switch (e) {
            case '"': out += '"'; break;
            case '\\': out += '\\'; break;
            case '/': out += '/'; break;
            case 'b': out += '\b'; break;
            case 'f': out += '\f'; break;
            case 'n': out += '\n'; break;
            case 'r': out += '\r'; break;
            case 't': out += '\t'; break;
            case 'u': {
                uint32_t cp = hex4(c);
                if (cp >= 0xD800 && cp < 0xDC00 && c.i + 1 < c.s.size() && c.s[c.i] == '\\' && c.s[c.i + 1] == 'u') {
                    c.i += 2;
                    const uint32_t lo = hex4(c);
                    cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                }
                append_utf8(out, cp);
                break;
            }
            default: c.fail("unknown escape");
        }
    }
}

// Skips a value that is not a plain number (nested objects / arrays / strings / literals): such entries are
// ignored, as upstream ignores values that are not numbers.
void skip_value(JsonCursor& c) {
    const char ch = c.peek();
    if (ch == '"') {
        parse_string(c);
    } else if (ch == '{' || ch == '[') {
        const char close = ch == '{' ? '}' : ']';
        ++c.i;
        while (c.peek() != close) {
            if (ch == '{') {
                parse_string(c);
                c.expect(':');
            }
            skip_value(c);
            if (c.peek() == ',') ++c.i;
        }
        ++c.i;
    } else {
        while (c.i < c.s.size() && c.s[c.i] != ',' && c.s[c.i] != '}' && c.s[c.i] != ']') ++c.i;
    }
}

template <typename F>
void for_each_number_entry(const std::string& text, F&& f) {
    JsonCursor c{text};
    c.expect('{');
    if (c.peek() == '}') return;
    for (;;) {
        std::string key = parse_string(c);
        c.expect(':');
        const char ch = c.peek();
        if (ch == '-' || (ch >= '0' && ch <= '9')) {
            size_t used = 0;
            double v = 0;
            try {
                v = std::stod(c.s.substr(c.i, 32), &used);
            } catch (const std::exception&) {
                c.fail("bad number");
            }
            c.i += used;
            f(key, int(v));
        } else {
            skip_value(c);
        }
        if (c.peek() == ',') {
            ++c.i;
            continue;
        }
        c.expect('}');
        return;
    }
}

// ---- binary stream helpers (32-bit counts and lengths, raw bytes) ----

void put_int(std::ostream& out, int v) { out.write(reinterpret_cast<const char*>(&v), sizeof(v)); }
void put_str(std::ostream& out, const std::string& s) {
    put_int(out, int(s.size()));
    out.write(s.data(), std::streamsize(s.size()));
}
int get_int(std::istream& in) {
    int v = 0;
    in.read(reinterpret_cast<char*>(&v), sizeof(v));
    if (!in) throw std::runtime_error("VocabLoader::load: truncated stream");
    return v;
}
std::string get_str(std::istream& in) {
    const int n = get_int(in);
    if (n < 0 || n > (1 << 24)) throw std::runtime_error("VocabLoader::load: bad string length");
    std::string s(size_t(n), '\0');
    in.read(&s[0], n);
    if (!in) throw std::runtime_error("VocabLoader::load: truncated stream");
    return s;
}

std::string directory_of(const std::string& path) {
    const size_t slash = path.find_last_of("/\\");
    return slash == std::string::npos ? std::string() : path.substr(0, slash + 1);
}

}  // namespace

VocabLoader::VocabLoader() { initialize_byte_to_unicode(); }
VocabLoader::~VocabLoader() = default;

// Printable ASCII (letters, digits, space, punctuation 0x20-0x7E) keeps its value; every other byte b is given
// the code point b + 256 (upstream vocab_loader.cu:20-43).
void VocabLoader::initialize_byte_to_unicode() {
    for (int b = 0; b < 256; ++b) {
        const int cp = (b >= 0x20 && b <= 0x7E) ? b : b + 256;
        byte_to_unicode_[b] = cp;
        unicode_to_byte_[cp] = b;
    }
}

void VocabLoader::add_token(const std::string& token) {
    if (token_to_index_.count(token)) return;
    token_to_index_[token] = int(index_to_token_.size());
    index_to_token_.push_back(token);
}

void VocabLoader::add_token(const std::string& token, int id) {
    if (token_to_index_.count(token) || id < 0) return;
    if (id >= int(index_to_token_.size())) index_to_token_.resize(size_t(id) + 1);
    token_to_index_[token] = id;
    index_to_token_[size_t(id)] = token;
}

int VocabLoader::token_to_id(const std::string& token) const {
    auto it = token_to_index_.find(token);
    if (it != token_to_index_.end()) return it->second;
    auto unk = token_to_index_.find("<|unk|>");
    // upstream recurses into get_unk_token_id() here, which never returns when "<|unk|>" itself is missing; a
    // vocabulary without it answers -1 instead
    return unk != token_to_index_.end() ? unk->second : -1;
}

std::string VocabLoader::id_to_token(int id) const {
    if (id >= 0 && id < int(index_to_token_.size())) return index_to_token_[size_t(id)];
    return "<|endoftext|>";
}

int VocabLoader::size() const { return int(index_to_token_.size()); }

void VocabLoader::clear() {
    token_to_index_.clear();
    index_to_token_.clear();
    bpe_merges_.clear();
}

void VocabLoader::load_from_file(const std::string& path) {
    clear();
    std::ifstream file(path);
    if (!file.is_open()) throw std::runtime_error("Could not open vocabulary file: " + path);
    std::stringstream buffer;
    buffer << file.rdbuf();
    const std::string text = buffer.str();
    add_token("<|endoftext|>");
    add_token("<|unk|>");
    add_token("<|pad|>");
    for_each_number_entry(text, [this](const std::string& token, int id) {
        if (id < 0) return;
        token_to_index_[token] = id;  // the file's id wins over the provisional special-token ids
        if (size_t(id) >= index_to_token_.size()) index_to_token_.resize(size_t(id) + 1);
        index_to_token_[size_t(id)] = token;
    });
    if (token_to_index_.empty()) throw std::runtime_error("Vocabulary file is empty or invalid");
    const std::string merges = directory_of(path) + "merges.txt";
    if (std::ifstream(merges).is_open()) load_bpe_merges(merges);
}

// One rule per line, "left right"; '#' lines and lines without a space are skipped (upstream :144-172).
void VocabLoader::load_bpe_merges(const std::string& path) {
    std::ifstream file(path);
    if (!file.is_open()) throw std::runtime_error("Could not open BPE merges file: " + path);
    std::string line;
    while (std::getline(file, line)) {
        if (line.empty() || line[0] == '#') continue;
        const size_t space = line.find(' ');
        if (space == std::string::npos) continue;
        const std::string left = line.substr(0, space), right = line.substr(space + 1);
        bpe_merges_.emplace_back(left + " " + right, left + right);
    }
}

const std::vector<std::pair<std::string, std::string>>& VocabLoader::get_bpe_merges() const { return bpe_merges_; }

void VocabLoader::save(std::ostream& out) const {
    put_int(out, int(token_to_index_.size()));
    for (const auto& kv : token_to_index_) {
        put_str(out, kv.first);
        put_int(out, kv.second);
    }
    put_int(out, int(index_to_token_.size()));
    for (const std::string& t : index_to_token_) put_str(out, t);
    put_int(out, int(bpe_merges_.size()));
    for (const auto& m : bpe_merges_) {
        put_str(out, m.first);
        put_str(out, m.second);
    }
    for (const auto* table : {&byte_to_unicode_, &unicode_to_byte_}) {
        put_int(out, int(table->size()));
        for (const auto& kv : *table) {
            put_int(out, kv.first);
            put_int(out, kv.second);
        }
    }
}

void VocabLoader::load(std::istream& in) {
    auto count = [&in]() {
        const int n = get_int(in);
        if (n < 0 || n > (1 << 26)) throw std::runtime_error("VocabLoader::load: bad count");
        return n;
    };
    token_to_index_.clear();
    for (int i = 0, n = count(); i < n; ++i) {
        std::string key = get_str(in);
        token_to_index_[key] = get_int(in);
    }
    index_to_token_.assign(size_t(count()), std::string());
    for (std::string& t : index_to_token_) t = get_str(in);
    bpe_merges_.assign(size_t(count()), {});
    for (auto& m : bpe_merges_) {
        m.first = get_str(in);
        m.second = get_str(in);
    }
    for (auto* table : {&byte_to_unicode_, &unicode_to_byte_}) {
        table->clear();
        for (int i = 0, n = count(); i < n; ++i) {
            const int key = get_int(in);
            (*table)[key] = get_int(in);
        }
    }
}

}  // namespace dnn
