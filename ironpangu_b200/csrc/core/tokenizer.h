// Tokenizers of the HTTP front end and the chat-prompt renderer.
//
//   ByteTokenizer   ids 0 pad, 1 bos, 2 eos, 3 + byte: no files needed (tests, synthetic models)
//   BpeTokenizer    byte-level BPE read from a Hugging Face `tokenizer.json` (model.type "BPE" with a ByteLevel pre-tokenizer /
//                   decoder, the format of the GPT-2, Qwen and Llama-3 families): vocabulary, ranked merges, added and special
//                   tokens. Text is first cut at added tokens (longest match), then into words by the family's splitting rule
//                   (contractions, an optional leading non-letter glued to a run of letters, single digits, punctuation runs
//                   with their trailing newlines, whitespace runs that leave one blank for the next word), every word is mapped
//                   byte by byte to the 256 printable stand-in characters and merged by rank. Decoding maps the stand-ins back to
//                   bytes, so encode -> decode is the identity on any byte string. Letters and digits beyond ASCII are
//                   classified by Unicode block (see `is_letter`), not by the full Unicode tables: word boundaries in text that
//                   mixes scripts and symbols can differ from the reference implementation's, ids never fail to round-trip.
//   Detokenizer     incremental: feeds ids, emits only complete UTF-8 sequences (a multi-byte character split across tokens is
//                   held back until its last byte arrives)
//   render_chat     messages -> prompt text: `chatml` (<|im_start|>role\ncontent<|im_end|>\n ... <|im_start|>assistant\n), chosen
//                   when the vocabulary has those markers, else `plain` (<|role|>\ncontent\n ... <|assistant|>\n)
// Reference: vendor/rust/src/tokenizer/src/hf.rs (tokenizer.json loading), vendor/rust/src/chat/src/renderer (templates).
#pragma once
#include <memory>
#include <unordered_map>

#include "base.h"

namespace ifab::tok {

class Tokenizer {
 public:
  virtual ~Tokenizer() = default;
  virtual std::vector<uint32_t> encode(std::string_view text) const = 0;
  // bytes of one token (special tokens render as their text unless `skip_special`); unknown ids render as <|id|>
  virtual std::string piece(uint32_t id, bool skip_special = false) const = 0;
  virtual uint32_t vocab_size() const = 0;
  virtual int64_t bos() const = 0;     // -1: none
  virtual int64_t eos() const = 0;
  virtual int64_t token_id(std::string_view text) const = 0;   // id of an added / special token by its text, -1 when absent
  virtual std::string name() const = 0;
  std::string decode(const std::vector<uint32_t>& ids, bool skip_special = false) const;
};

class ByteTokenizer : public Tokenizer {
 public:
  static constexpr uint32_t kPad = 0, kBos = 1, kEos = 2, kFirstByte = 3, kVocab = 259;
  std::vector<uint32_t> encode(std::string_view text) const override;
  std::string piece(uint32_t id, bool skip_special = false) const override;
  uint32_t vocab_size() const override { return kVocab; }
  int64_t bos() const override { return kBos; }
  int64_t eos() const override { return kEos; }
  int64_t token_id(std::string_view) const override { return -1; }
  std::string name() const override { return "bytes"; }
};

class BpeTokenizer : public Tokenizer {
 public:
  // `json_text`: the contents of tokenizer.json (at most 64 MiB). Throws Invalid for other model types or malformed tables.
  explicit BpeTokenizer(std::string_view json_text);
  static std::shared_ptr<BpeTokenizer> from_file(const std::string& path);
  std::vector<uint32_t> encode(std::string_view text) const override;
  std::string piece(uint32_t id, bool skip_special = false) const override;
  uint32_t vocab_size() const override { return (uint32_t)pieces_.size(); }
  int64_t bos() const override { return bos_; }
  int64_t eos() const override { return eos_; }
  int64_t token_id(std::string_view text) const override;
  std::string name() const override { return "bpe"; }
  // the word splitter, exposed for tests
  static std::vector<std::string_view> split_words(std::string_view text);

 private:
  void encode_word(std::string_view word, std::vector<uint32_t>& out) const;
  std::unordered_map<std::string, uint32_t> vocab_;                  // stand-in text -> id
  std::vector<std::string> pieces_;                                  // id -> raw bytes
  std::vector<uint8_t> special_;                                     // id -> 1 when special
  std::unordered_map<std::string, uint32_t> ranks_;                  // "left right" -> rank
  std::vector<std::pair<std::string, uint32_t>> added_;              // added tokens, longest first
  mutable std::unordered_map<std::string, std::vector<uint32_t>> cache_;
  int64_t bos_ = -1, eos_ = -1;
};

class Detokenizer {
 public:
  explicit Detokenizer(std::shared_ptr<const Tokenizer> t, bool skip_special = true) : tok_(std::move(t)), skip_special_(skip_special) {}
  std::string feed(uint32_t id);
  std::string flush();

 private:
  std::shared_ptr<const Tokenizer> tok_;
  bool skip_special_;
  std::string pending_;
};

struct ChatMessage {
  std::string role, content;
};
// `style`: "auto" (chatml when the tokenizer knows <|im_start|> and <|im_end|>, else plain), "chatml" or "plain".
std::string render_chat(const std::vector<ChatMessage>& messages, const Tokenizer& tok, const std::string& style = "auto");

// "bytes" or a path to tokenizer.json
std::shared_ptr<Tokenizer> load_tokenizer(const std::string& spec);

// complete UTF-8 sequences at the front of `pending` are moved to the result; invalid bytes become U+FFFD; with `final`
// an incomplete tail is flushed as U+FFFD too
std::string drain_utf8(std::string& pending, bool final);

}  // namespace ifab::tok
