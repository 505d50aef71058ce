"""The byte-level BPE tokenizer of the server against the `tokenizers` library on a vocabulary the test trains itself."""
import json

import pytest

from ironpangu_b200 import compiler

tokenizers = pytest.importorskip("tokenizers")

SPLIT = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+")
CORPUS = ["hello world, hello there! it's 12345 o'clock\n\n  an indented line\tand a tab",
          "the quick brown fox jumps over the lazy dog; THE QUICK BROWN FOX",
          "def f(x):\n    return x + 1  # comment\n", "naïve café déjà vu — «quotes» … ¿qué?", "数字 123 と 日本語 のテキスト。中文也可以",
          "we've they'll I'm you'd can't WE'VE", "a  b   c    d\r\n\r\ne", "price: $4.50 (approx.) 100% sure!!!"] * 4
SAMPLES = ["hello  world's 42!\n x", "", " ", "  leading and trailing  ", "tabs\tand\nnewlines\r\n\r\n  done", "it's we've THEY'LL o'clock 'quoted'",
           "x=1;y=22;zzz=333", "naïve café — «ok» … 数字 12 日本語。", "emoji 🙂 and bytes é́", "<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n",
           "a<|endoftext|>b <|endoftext|>", "ünïcödé wörds", "mixed123abc 4 5  6", "\n\n\n", "trailing space \n"]


@pytest.fixture(scope="module")
def trained(tmp_path_factory):
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers, trainers

    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(SPLIT), behavior="isolated"),
                                                 pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok.decoder = decoders.ByteLevel()
    tr = trainers.BpeTrainer(vocab_size=700, special_tokens=["<|endoftext|>", "<|im_start|>", "<|im_end|>"],
                             initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(CORPUS, tr)
    path = tmp_path_factory.mktemp("tok") / "tokenizer.json"
    path.write_text(tok.to_str())
    return tok, path


def run(verb, path, payload, tmp_path, *extra):
    f = tmp_path / "in.txt"
    f.write_text(payload, encoding="utf-8", newline="")
    r = compiler.cli(verb, str(path), str(f), *extra)
    assert r.returncode == 0, r.stderr
    return json.loads(r.stdout)


def test_ids_equal_the_library_and_round_trip(trained, tmp_path):
    ref, path = trained
    for text in SAMPLES:
        got = run("tokenize", path, text, tmp_path)
        want = ref.encode(text)
        assert got["ids"] == want.ids, (text, got["words"], want.tokens)
        back = run("detokenize", path, json.dumps(got["ids"]), tmp_path)
        assert back["text"] == text
        assert "".join(back["stream"]) == text            # the incremental form emits the same text, in whole characters
    assert run("tokenize", path, "x", tmp_path)["vocab_size"] == ref.get_vocab_size()


def test_streaming_holds_back_split_characters(trained, tmp_path):
    ref, path = trained
    ids = ref.encode("🙂é").ids                       # four- and two-byte characters that the small vocabulary splits into bytes
    assert len(ids) >= 5
    parts = run("detokenize", path, json.dumps(ids), tmp_path)["stream"]
    assert "".join(parts) == "🙂é" and all(p in ("", "🙂", "é") for p in parts)
    special = run("detokenize", path, json.dumps(ref.encode("a<|endoftext|>b").ids), tmp_path)
    assert special["text"] == "a<|endoftext|>b" and special["text_without_special"] == "ab"
    unknown = run("detokenize", path, json.dumps([ids[0], 999999]), tmp_path)
    assert unknown["text"].endswith("<|999999|>")


def test_chat_rendering(trained, tmp_path):
    ref, path = trained
    msgs = json.dumps([{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}])
    out = run("render-chat", path, msgs, tmp_path)
    assert out["text"] == "<|im_start|>system\nbe brief<|im_end|>\n<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"
    assert out["ids"] == ref.encode(out["text"]).ids and out["ids"].count(ref.token_to_id("<|im_start|>")) == 3
    plain = run("render-chat", "bytes", msgs, tmp_path)
    assert plain["text"] == "<|system|>\nbe brief\n<|user|>\nhi\n<|assistant|>\n" and plain["tokenizer"] == "bytes"
    assert run("render-chat", path, msgs, tmp_path, "plain")["text"] == plain["text"]


def test_other_tokenizer_models_are_refused(tmp_path):
    bad = tmp_path / "tokenizer.json"
    bad.write_text(json.dumps({"model": {"type": "Unigram", "vocab": []}}))
    f = tmp_path / "t.txt"
    f.write_text("x")
    r = compiler.cli("tokenize", str(bad), str(f))
    assert r.returncode == 1 and "Unigram" in r.stderr
    bad.write_text(json.dumps({"model": {"type": "BPE", "vocab": {"a": 0}, "merges": []}, "pre_tokenizer": {"type": "Whitespace"}}))
    r = compiler.cli("tokenize", str(bad), str(f))
    assert r.returncode == 1 and "byte-level" in r.stderr


def test_server_speaks_the_trained_vocabulary(trained):
    """The HTTP front end with `--tokenizer tokenizer.json`: /tokenize and /detokenize use the BPE vocabulary, chat prompts are
    rendered with the vocabulary's own turn markers, and streamed text arrives in whole characters."""
    from test_server import Server

    ref, path = trained
    s = Server("--mock", "--tokenizer", str(path), "--max-num-seqs", "2", "--max-num-batched-tokens", "64", "--max-model-len", "256")
    try:
        text = "hello world's café 🙂"
        status, body = s.post("/tokenize", {"prompt": text})
        assert status == 200 and body["tokens"] == ref.encode(text).ids
        status, body = s.post("/detokenize", {"tokens": ref.encode(text).ids})
        assert status == 200 and body["prompt"] == text
        status, body = s.post("/tokenize", {"messages": [{"role": "user", "content": "hi"}]})
        assert status == 200 and body["tokens"] == ref.encode("<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n").ids
        status, body = s.post("/v1/chat/completions", {"model": "m", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 5})
        assert status == 200 and body["usage"]["prompt_tokens"] == len(ref.encode("<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n").ids)
        assert isinstance(body["choices"][0]["message"]["content"], str)
    finally:
        s.close()
