// BpeTokenizer: the text front end of the language models (upstream dnn/tokens/bpe_tokenizer.cuh:18-57).
//
// Behaviour is upstream's (dnn/tokens/bpe_tokenizer.cu), which its own tests pin
// (tests/tokens/bpe_tokenizer_test.cu:88-190):
//   encode   runs of white space and control characters become single separators; every word that is in the
//            vocabulary as a whole becomes its id, any other word is spelt out byte by byte (a byte that is not in
//            the vocabulary gives the unknown-token id); add_special_tokens brackets the ids with BOS / EOS.  The
//            merge rules the vocabulary carries are NOT applied by encode (upstream's apply_bpe_to_word is never
//            called: "helo" encodes as h, e, l, o with the test vocabulary although "he" is a token);
//   decode   concatenates the token strings (no separators are re-inserted) and drops BOS / EOS / UNK / PAD when
//            skip_special_tokens is set;
//   text_to_unicode / unicode_to_text   upstream narrows the mapped code point back to one char, which makes
//            both directions the identity on bytes; kept, so that ids agree with upstream's for any input.
// merge_word() is an addition: it applies the merge rules to one word the way upstream's private, unused
// apply_bpe_to_word does (first rule in file order that matches any adjacent pair, repeated until none does).
#pragma once

#include <memory>
#include <string>
#include <vector>

#include "dnn/tokens/tokenizer.cuh"
#include "dnn/tokens/vocab_loader.cuh"

namespace dnn {

class BpeTokenizer : public Tokenizer {
public:
    explicit BpeTokenizer(std::shared_ptr<VocabLoader> vocab);  // throws std::invalid_argument on null

    std::vector<int> encode(const std::string& text, bool add_special_tokens = false) const override;
    std::string decode(const std::vector<int>& token_ids, bool skip_special_tokens = true) const override;

    int get_bos_token_id() const override { return vocab_->get_bos_token_id(); }
    int get_eos_token_id() const override { return vocab_->get_eos_token_id(); }
    int get_unk_token_id() const override { return vocab_->get_unk_token_id(); }
    int get_pad_token_id() const override { return vocab_->get_pad_token_id(); }
    int vocab_size() const override { return vocab_->size(); }

    void save(std::ostream& out) const override;
    void load(std::istream& in) override;

    std::string text_to_unicode(const std::string& text) const;
    std::string unicode_to_text(const std::string& unicode) const;

    std::vector<std::string> merge_word(const std::string& word) const;

private:
    std::shared_ptr<VocabLoader> vocab_;
    std::string clean_text(const std::string& text) const;
};

}  // namespace dnn
