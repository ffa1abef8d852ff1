// Tokenizer: the abstract text <-> token-id interface the language models hold (upstream
// dnn/tokens/tokenizer.cuh).  The implementation that ships with it is BpeTokenizer (bpe_tokenizer.cuh).
#pragma once

#include <iostream>
#include <string>
#include <vector>

namespace dnn {

class Tokenizer {
public:
    virtual ~Tokenizer() = default;
    virtual std::vector<int> encode(const std::string& text, bool add_special_tokens = false) const = 0;
    virtual std::string decode(const std::vector<int>& token_ids, bool skip_special_tokens = true) const = 0;
    virtual int get_bos_token_id() const = 0;
    virtual int get_eos_token_id() const = 0;
    virtual int get_unk_token_id() const = 0;
    virtual int get_pad_token_id() const = 0;
    virtual int vocab_size() const = 0;
    virtual void save(std::ostream& out) const = 0;
    virtual void load(std::istream& in) = 0;
};

}  // namespace dnn
