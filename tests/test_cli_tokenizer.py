"""Command line decisions that need no GPU, and the byte-level BPE tokenizer."""
import json
import subprocess
import sys
from pathlib import Path

from oracle_engine_b200.tokenizer.bpe import Tokenizer, _byte_tables

ROOT = Path(__file__).resolve().parent.parent


def _run(*args):
    return subprocess.run([sys.executable, str(ROOT / "bin" / "oracle"), *args], capture_output=True, text=True)


def test_cli_usage_and_exit_codes(tmp_path):
    r = _run("-h")
    assert r.returncode == 0 and "Usage:" in r.stderr and "--temp" in r.stderr
    assert _run("--frobnicate").returncode == 2
    r = _run("-m")
    assert r.returncode == 2 and "missing value after -m" in r.stderr
    assert _run("-m", "x").returncode == 2                      # no prompt
    assert _run("-p", "hi").returncode == 2                     # no model
    assert _run("-m", "x", "--tokens", "1,b").returncode == 2   # bad value
    r = _run("-m", str(tmp_path / "nothing"), "--tokens", "1,2")
    assert r.returncode == 1 and "failed to load model" in r.stderr


def _toy_tokenizer(tmp_path):
    b2u, _ = _byte_tables()
    sp = b2u[ord(" ")]
    vocab = {ch: i for i, ch in enumerate(sorted(set(b2u[b] for b in range(256))))}
    for t in ("he", "ll", "hell", "hello", sp + "w", sp + "wo"):
        vocab[t] = len(vocab)
    merges = ["h e", "l l", "he ll", "hell o", f"{sp} w", f"{sp}w o"]
    raw = {"model": {"vocab": vocab, "merges": merges},
           "added_tokens": [{"id": 900, "content": "<|eot|>", "special": True}]}
    (tmp_path / "tokenizer.json").write_text(json.dumps(raw))
    return Tokenizer.from_folder(tmp_path, bos_id=7), vocab, sp


def test_bpe_merges_by_rank_and_round_trips(tmp_path):
    tok, vocab, sp = _toy_tokenizer(tmp_path)
    ids = tok.encode("hello world", add_bos=True)
    assert ids[0] == 7
    assert ids[1] == vocab["hello"]                                          # h e | l l | he ll | hell o
    assert ids[2] == vocab[sp + "wo"] and [tok.id2tok[i] for i in ids[3:]] == ["r", "l", "d"]
    assert tok.decode(ids[1:]) == "hello world"
    text = "héllo\n wörld\t!\n<|eot|> ok"
    ids = tok.encode(text, add_bos=False)
    assert 900 in ids                                                        # a special token as a whole word
    assert tok.decode(ids) == text.replace("<|eot|>", "")                    # special tokens are not shown
    assert tok.encode("", add_bos=False) == []
    assert Tokenizer.from_folder(tmp_path / "none") is None
