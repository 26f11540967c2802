"""The optional tokenizer, the text streamer and the command line's options."""
import json

import pytest

from velomind_b200.api import TextStreamer
from velomind_b200.cli import build_parser
from velomind_b200.tokenizer import ByteLevelBPETokenizer, _BYTE_TO_UNI, pretokenize


def _tokenizer_json(tmp_path):
    vocab = {ch: i for i, ch in enumerate(_BYTE_TO_UNI[b] for b in range(256))}
    merges = [("h", "e"), ("l", "l"), ("he", "ll"), ("hell", "o"), ("Ġ", "w"), ("Ġw", "o")]
    for a, b in merges:
        vocab[a + b] = len(vocab)
    root = {"model": {"vocab": vocab, "merges": [f"{a} {b}" for a, b in merges]},
            "added_tokens": [{"id": 300, "content": "<|endoftext|>"}, {"id": 301, "content": "<|im_end|>"}]}
    p = tmp_path / "tokenizer.json"
    p.write_text(json.dumps(root))
    return str(p), vocab


def test_pretokenizer_pieces():
    u = lambda s: "".join(_BYTE_TO_UNI[b] for b in s.encode())
    assert pretokenize("hello world") == [u("hello"), u(" world")]
    assert pretokenize("it's 42!") == [u("it"), u("'s"), u(" "), u("4"), u("2"), u("!")]
    assert pretokenize("a  b\n") == [u("a"), u("  "), u("b"), u("\n")]
    assert pretokenize("we'll…ok") == [u("we"), u("'ll"), u("…"), u("ok")]


def test_bpe_round_trip_and_special_ids(tmp_path):
    path, vocab = _tokenizer_json(tmp_path)
    tok = ByteLevelBPETokenizer.from_file(path)
    assert tok.bos_id == 300 and tok.eos_id == 301 and tok.pad_id is None
    ids = tok.encode("hello world")
    assert ids[0] == vocab["hello"] and ids[1] == vocab["Ġwo"] and len(ids) == 5
    for text in ["hello world", "héllo wörld 123", "it's\n  fine…", "日本語 ok"]:
        assert tok.decode(tok.encode(text)) == text
    assert tok.decode([300] + tok.encode("hello") + [301]) == "hello"        # begin/end ids are skipped
    assert tok.encode("") == []
    with pytest.raises(ValueError, match="model.vocab"):
        bad = tmp_path / "bad.json"; bad.write_text("{}"); ByteLevelBPETokenizer.from_file(str(bad))


def test_streamer_emits_deltas_and_waits_for_whole_characters(tmp_path):
    path, _ = _tokenizer_json(tmp_path)
    tok = ByteLevelBPETokenizer.from_file(path)
    text = "hello wörld日本"
    ids = tok.encode(text)
    st = TextStreamer(tok)
    pieces = [st.put(i) for i in ids]
    assert "".join(pieces) + st.flush() == text
    assert "" in pieces                                   # the bytes of a multi-byte character arrive one token at a time
    assert all("�" not in p for p in pieces)
    assert TextStreamer(None).put(17) == "[17]"           # without a tokenizer: the id in brackets


def test_cli_options_have_the_reference_names_and_defaults():
    a = build_parser().parse_args([])
    assert (a.temp, a.top_p, a.max_tokens, a.prompt, a.synthetic, a.device) == (0.7, 0.9, 32, "", False, "cuda:0")
    a = build_parser().parse_args(["--model", "m", "--tokenizer", "t.json", "--temp", "0", "--top-p", "0.5", "--max-tokens", "7",
                                   "--prompt", "hi", "--synthetic", "--device", "cuda"])
    assert (a.model, a.tokenizer, a.temp, a.top_p, a.max_tokens, a.prompt, a.synthetic) == ("m", "t.json", 0.0, 0.5, 7, "hi", True)


# ------------------------------------------------------------------------------------------ the `>>>` loop's commands
class _FakeResult:
    def __init__(self, tokens):
        self.tokens = tokens


class _FakeEngine:
    """Stands in for TextEngine in the console: answers a text prompt with its length as words, records what it was asked."""

    def __init__(self, tokenizer=True):
        self.tokenizer = object() if tokenizer else None
        self.asked = []

    def generate(self, prompts, temperature, top_p, max_tokens, seed, on_token):
        self.asked.append((prompts[0], temperature, top_p, max_tokens, seed))
        for i, piece in enumerate(("re", "ply")):
            on_token(0, 100 + i, piece)
        return [_FakeResult([100, 101])]

    def describe(self):
        return {"Backend": "cuda:0", "Hidden": 576}


def _console(tokenizer=True):
    from velomind_b200.cli import Console
    args = build_parser().parse_args(["--synthetic"])
    said = []
    return Console(_FakeEngine(tokenizer), args, out=said.append), args, said


def test_console_commands_change_the_sampling_state(capsys):
    c, args, said = _console()
    assert c.command("/temp 0.25") is True and args.temp == 0.25 and "Temperature set to 0.25" in said[-1]
    assert c.command("/top_p 0.5") is True and args.top_p == 0.5
    assert c.command("/max 7") is True and args.max_tokens == 7
    assert c.command("/temp x") is True and args.temp == 0.25 and "Invalid" in said[-1]
    assert c.command("/max -3") is True and args.max_tokens == 7 and "Invalid" in said[-1]
    assert c.command("/help") is True and any("/save <file>" in s for s in said) and any("Current: 0.25" in s for s in said)
    assert c.command("/model") is True and any(s.startswith("Hidden:") for s in said)
    assert c.command("hello") is None and c.command("/nonsense") is None        # not commands: prompts
    assert c.command("/exit") is False and c.command("/quit") is False


def test_console_composes_the_conversation_and_moves_the_seed(capsys, tmp_path):
    c, args, said = _console()
    c.command("/system be brief")
    c.turn("first question")
    assert c.engine.asked[-1] == ("be brief\nfirst question", 0.7, 0.9, 32, 42)
    c.turn("second")
    assert c.engine.asked[-1][0] == "be brief\nfirst question\nreply\nsecond" and c.engine.asked[-1][4] == 43
    c.command("/history")
    assert "2 tokens" in said[-1] and "Last text: reply" in said[-1]
    path = str(tmp_path / "talk.txt")
    assert c.command(f"/save {path}") is True and "Saved to" in said[-1]
    c.command("/clear")
    assert c.turns == [] and c.system == "be brief"
    c.command("/system")
    assert c.system == ""
    assert c.command(f"/load {path}") is True and "(4 turns)" in said[-1]
    assert c.system == "be brief" and c.turns == ["first question", "reply", "second", "reply"]
    assert c.command(f"/load {path}.missing") is True and "Load failed" in said[-1]


def test_console_without_a_tokenizer_takes_token_ids(capsys):
    c, args, said = _console(tokenizer=False)
    c.turn("1, 5 17")
    assert c.engine.asked[-1][0] == [1, 5, 17] and c.turns == []
    c.turn("words")
    assert "token ids" in said[-1] and len(c.engine.asked) == 1
