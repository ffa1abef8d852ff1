"""The text front end (dnn::VocabLoader, dnn::BpeTokenizer) on the CPU: the upstream project's own test cases
(tests/tokens/vocab_loader_test.cu, tests/tokens/bpe_tokenizer_test.cu), restated in C++ in the harness library."""
import ctypes as C


def test_tokenizer_and_vocabulary_cases(df8, tmp_path):
    lib = df8.dnn_lib()
    buf = C.create_string_buffer(1 << 14)
    failures = lib.dnn_selftest_tokenizer(str(tmp_path).encode(), buf, len(buf))
    assert failures == 0, buf.value.decode()



def test_tokenizer_harness_round_trip(df8, tmp_path):
    """encode / decode / saved state through the C harness (what a Python caller uses)."""
    import json

    vocab = {"<|endoftext|>": 0, "<|unk|>": 1, "<|pad|>": 2, "the": 3, "quick": 4, "t": 5, "h": 6, "e": 7, "Hello,": 8}
    (tmp_path / "vocab.json").write_text(json.dumps(vocab))
    path = str(tmp_path / "vocab.json").encode()
    state = str(tmp_path / "state.bin").encode()
    lib = df8.dnn_lib()
    assert lib.dnn_tokenizer_save(path, state) == 0
    for text, want in [("the quick  teh", [3, 4, 5, 7, 6]), ("Hello, the", [8, 3]), ("zz", [1, 1]), ("", [])]:
        for vocab_arg, state_arg in ((path, b""), (b"", state)):
            ids = (C.c_int * 64)()
            n = lib.dnn_tokenizer_encode(vocab_arg, state_arg, text.encode(), 1, ids, 64)
            assert n == len(want) + 2 and list(ids[:n]) == [0] + want + [0], (text, list(ids[:n]))
            out = C.create_string_buffer(256)
            m = lib.dnn_tokenizer_decode(vocab_arg, state_arg, ids, n, 1, out, 256)
            assert out.raw[:m].decode() == "".join(t for t in text.split() if t in vocab or True).replace("z", "")
    assert lib.dnn_tokenizer_encode(b"/nonexistent/vocab.json", b"", b"x", 0, (C.c_int * 4)(), 4) == -1
