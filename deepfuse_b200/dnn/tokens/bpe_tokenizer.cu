#include "dnn/tokens/bpe_tokenizer.cuh"

#include <cctype>
#include <stdexcept>

namespace dnn {

namespace {
// what std::isspace calls white space in the "C" locale, on an unsigned value
bool is_space(unsigned char c) { return c == ' ' || (c >= '\t' && c <= '\r'); }
}  // namespace

BpeTokenizer::BpeTokenizer(std::shared_ptr<VocabLoader> vocab) : vocab_(std::move(vocab)) {
    if (!vocab_) throw std::invalid_argument("VocabLoader cannot be null");
}

// Each byte goes through the vocabulary's byte table and the result is narrowed to one char again, which maps a
// byte b to b (printable) or to (b + 256) mod 256 = b: the identity (upstream :18-29).
std::string BpeTokenizer::text_to_unicode(const std::string& text) const {
    const auto& table = vocab_->bytes_to_unicode();
    std::string out;
    out.reserve(text.size());
    for (unsigned char c : text) {
        auto it = table.find(c);
        out += it != table.end() ? static_cast<char>(it->second) : static_cast<char>(c);
    }
    return out;
}

std::string BpeTokenizer::unicode_to_text(const std::string& unicode) const {
    const auto& table = vocab_->unicode_to_bytes();
    std::string out;
    out.reserve(unicode.size());
    for (unsigned char c : unicode) {
        auto it = table.find(c);
        out += it != table.end() ? static_cast<char>(it->second) : static_cast<char>(c);
    }
    return out;
}

// Runs of white space collapse to one space; bytes below 0x20, 0x7F and (as signed chars) every byte above 0x7F
// turn into spaces; the ends are trimmed (upstream :44-65).
std::string BpeTokenizer::clean_text(const std::string& text) const {
    std::string out;
    out.reserve(text.size());
    bool in_space = false;
    for (unsigned char c : text) {
        if (is_space(c)) {
            if (!in_space) out += ' ';
            in_space = true;
            continue;
        }
        in_space = false;
        out += (c >= 0x20 && c < 0x7F) ? static_cast<char>(c) : ' ';
    }
    const size_t first = out.find_first_not_of(" \t\n\r\f\v");
    if (first == std::string::npos) return std::string();
    const size_t last = out.find_last_not_of(" \t\n\r\f\v");
    return out.substr(first, last - first + 1);
}

std::vector<int> BpeTokenizer::encode(const std::string& text, bool add_special_tokens) const {
    std::vector<int> ids;
    if (add_special_tokens) ids.push_back(get_bos_token_id());
    const std::string prepared = text_to_unicode(clean_text(text));
    const int unk = vocab_->get_unk_token_id();
    size_t i = 0;
    while (i < prepared.size()) {
        while (i < prepared.size() && is_space(static_cast<unsigned char>(prepared[i]))) ++i;
        size_t j = i;
        while (j < prepared.size() && !is_space(static_cast<unsigned char>(prepared[j]))) ++j;
        if (j == i) break;
        const std::string word = prepared.substr(i, j - i);
        const int whole = vocab_->token_to_id(word);
        if (whole != unk) {
            ids.push_back(whole);
        } else {
            for (char c : word) ids.push_back(vocab_->token_to_id(std::string(1, c)));  // unknown bytes give `unk`
        }
        i = j;
    }
    if (add_special_tokens) ids.push_back(get_eos_token_id());
    return ids;
}

std::string BpeTokenizer::decode(const std::vector<int>& token_ids, bool skip_special_tokens) const {
    const int bos = get_bos_token_id(), eos = get_eos_token_id(), unk = get_unk_token_id(), pad = get_pad_token_id();
    std::string text;
    for (int id : token_ids) {
        if (skip_special_tokens && (id == bos || id == eos || id == unk || id == pad)) continue;
        const std::string token = vocab_->id_to_token(id);
        if (token == "<|endoftext|>") continue;
        text += token;
    }
    return unicode_to_text(text);
}

std::vector<std::string> BpeTokenizer::merge_word(const std::string& word) const {
    std::vector<std::string> parts;
    for (char c : word) parts.emplace_back(1, c);
    bool merged = true;
    while (merged && parts.size() > 1) {
        merged = false;
        for (const auto& rule : vocab_->get_bpe_merges()) {
            for (size_t i = 0; i + 1 < parts.size(); ++i) {
                // a rule is stored as ("left right", "leftright")
                if (parts[i] + " " + parts[i + 1] == rule.first) {
                    parts[i] = rule.second;
                    parts.erase(parts.begin() + long(i) + 1);
                    merged = true;
                    break;
                }
            }
            if (merged) break;
        }
    }
    return parts;
}

void BpeTokenizer::save(std::ostream& out) const { vocab_->save(out); }
void BpeTokenizer::load(std::istream& in) { vocab_->load(in); }

}  // namespace dnn
