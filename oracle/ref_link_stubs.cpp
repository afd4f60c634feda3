// TEST INFRASTRUCTURE — link stub for the one class of the reference that cannot be compiled
// here: Gpt2Tokenizer (src/gpt2_tokenizer.cpp needs the PCRE2 library, which this build
// environment lacks). The reference's src/generate.cpp refers to it only from its GPT-2 text
// codec; the link check drives generate_tokens and run_training with token ids directly, so no
// tokenizer member is ever called. Every member throws, to make an accidental call visible.
#include <stdexcept>

#include "gpt2_tokenizer.hpp"

struct Gpt2Tokenizer::Regex {};

Gpt2Tokenizer::Gpt2Tokenizer() = default;
Gpt2Tokenizer::~Gpt2Tokenizer() = default;

void Gpt2Tokenizer::load(const std::string&, const std::string&) {
  throw std::runtime_error("Gpt2Tokenizer is a link stub in this check (no PCRE2 here)");
}
std::vector<uint16_t> Gpt2Tokenizer::encode(const std::string&) const {
  throw std::runtime_error("Gpt2Tokenizer is a link stub in this check (no PCRE2 here)");
}
std::string Gpt2Tokenizer::decode(const std::vector<uint16_t>&) const {
  throw std::runtime_error("Gpt2Tokenizer is a link stub in this check (no PCRE2 here)");
}
