"""Stop strings with hold-back, whole UTF-8 characters, and cancelling a request: the two state
machines alone (the cases of hostfog/hfee internal/llm/text_test.go:5-40), the per-request text
stream over a fake tokenizer, and generation over the CPU doubles of the kernels that stops in the
middle, is cancelled from a callback or through the ``cancel`` set, pipelined and step by step."""
import numpy as np
import pytest

import plain_llama as plain
from hfee_b200.engine.text import Stopper, TextStream, TokenizerAdapter, Utf8Buffer


# ---------------------------------------------------------------- text_test.go:5-40
def test_stopper_withholds_and_never_emits_the_stop_string():
    s = Stopper(["</end>"])
    out = ""
    for piece in ["Hello", " wor", "ld</", "en", "d> ignored"]:
        text, hit = s.push(piece)
        out += text
        if hit:
            break
    assert hit and out == "Hello world"


def test_stopper_flushes_a_partial_match():
    s = Stopper(["STOP"])
    text, hit = s.push("go ST")
    assert (text, hit) == ("go ", False)
    assert s.flush() == "ST"


def test_utf8_buffer_holds_back_half_a_character():
    b = Utf8Buffer()
    euro = "€".encode()
    assert b.add(euro[:2]) == ""
    assert b.add(euro[2:]) == "€"


def test_stopper_with_several_stops_holds_the_longest_possible_prefix():
    s = Stopper(["abcX", "cdY", ""])
    assert s.push("12abc") == ("12", False)         # "abc" may become "abcX"
    assert s.push("d") == ("ab", False)             # "abcd" cannot; "cd" may become "cdY"
    assert s.push("Y tail") == ("", True)
    assert s.flush() == ""


# ---------------------------------------------------------------- a fake tokenizer
class ByteTokenizer:
    """Token id -> a fixed piece of bytes (like the reference's Tokenizer.Piece)."""

    def __init__(self, pieces):
        self.pieces = [p if isinstance(p, bytes) else p.encode() for p in pieces]

    def piece(self, token):
        return self.pieces[token % len(self.pieces)]

    def decode(self, ids):
        return b"".join(self.piece(t) for t in ids).decode("utf-8", errors="replace")

    def encode(self, text):
        raise NotImplementedError


class DecodeOnlyTokenizer:
    """The same without single-token pieces: only decode(ids), as a tokenizers.Tokenizer has."""

    def __init__(self, pieces):
        self._t = ByteTokenizer(pieces)

    def decode(self, ids):
        return self._t.decode(ids)

    def encode(self, text):
        raise NotImplementedError


@pytest.mark.parametrize("kind", [ByteTokenizer, DecodeOnlyTokenizer])
def test_text_stream_characters_leading_spaces_and_whole_tokens(kind):
    euro = "€".encode()
    tok = TokenizerAdapter(kind([" ", " He", "llo", euro[:1], euro[1:], " wor", "ld</", "en", "d> ignored", "!"]))
    st = TextStream(tok, ["</end>"])
    outs = [st.push(i) for i in range(9)]
    assert [o for o, _ in outs[:3]] == ["", "He", "llo"]            # leading spaces of the answer are dropped
    assert outs[3][0] == "" and outs[4][0] == "€"                   # half a character is held back
    assert "".join(o for o, _ in outs) == "Hello€ world" and outs[8][1] and not outs[7][1]
    assert st.text == "Hello€ world" and st.finish() == ""
    assert st.whole_tokens == 6                                      # "ld</" is cut by the stop string
    st2 = TextStream(tok, ["</x"])
    for i in (1, 2, 6):
        st2.push(i)
    assert st2.text == "Hellold" and st2.whole_tokens == 2           # "</" may become the stop string
    assert st2.finish() == "</" and st2.whole_tokens == 3            # it did not: released at the end


def test_text_stream_stop_inside_the_characters_of_the_last_token():
    tok = TokenizerAdapter(ByteTokenizer(["ab", "cS", "TOP"]))
    st = TextStream(tok, ["STOP"])
    assert st.push(0) == ("ab", False) and st.push(1) == ("c", False) and st.push(2) == ("", True)
    assert st.whole_tokens == 1


# ---------------------------------------------------------------- generation over the CPU doubles
LETTERS = [chr(ord("a") + i % 26) + (chr(ord("A") + (i // 26) % 26) if i % 3 == 0 else "") for i in range(256)]


def _engine(tiny_dirs, pipeline, **kw):
    from hfee_b200 import Engine
    settings = dict(dtype="float32", page_size=16, max_requests=3, max_context=128, max_batch_tokens=64, device="cpu")
    settings.update(kw)
    eng = Engine(tiny_dirs["A"], tokenizer=ByteTokenizer(LETTERS), **settings)
    eng.pipeline = pipeline
    return eng


def _all_free(eng):
    eng.runner.cache.check_invariants()
    return eng.runner.cache.free_pages() == eng.runner.cache.num_pages and \
        eng.runner.cache.free_slots() == eng.runner.cache.max_requests


@pytest.mark.parametrize("pipeline", [True, False])
def test_generation_stops_at_a_stop_string_in_the_middle(tiny_dirs, cpu_ops, pipeline):
    from hfee_b200 import SamplingOptions
    cfg, w = plain.load_model_dir(tiny_dirs["A"])
    rng = np.random.default_rng(21)
    prompts = [rng.integers(0, cfg.vocab, size=n).tolist() for n in (20, 25, 30)]
    want = [plain.greedy_generate(cfg, w, p, 16) for p in prompts]
    texts = ["".join(LETTERS[t] for t in wnt) for wnt in want]
    # a stop string for request 0 that begins inside its 7th token's text or right behind it, and spans tokens
    ends = np.cumsum([len(LETTERS[t]) for t in want[0]])
    at = int(ends[6]) - 1 if len(LETTERS[want[0][6]]) == 2 else int(ends[6])
    stop = texts[0][at:at + 3]
    assert texts[0].find(stop) == at
    opts = [SamplingOptions.greedy(num_predict=16).with_(stop=[stop]), SamplingOptions.greedy(num_predict=16),
            SamplingOptions.greedy(num_predict=16).with_(stop=["\x00never"])]
    eng = _engine(tiny_dirs, pipeline)
    seen_tokens = [[] for _ in prompts]
    seen_text = ["" for _ in prompts]

    def on_token(i, t):
        seen_tokens[i].append(t)

    def on_text(i, s):
        seen_text[i] += s

    res = eng.generate(prompts, opts, on_token=on_token, on_text=on_text)
    whole = int(np.searchsorted(ends, at, side="right"))                  # tokens that end at or before the stop string
    assert res[0].text == texts[0][:at] and seen_text[0] == texts[0][:at] and stop not in seen_text[0]
    assert res[0].token_ids == want[0][:whole] and seen_tokens[0] == want[0][:whole]
    assert res[0].stats.done_reason == "stop"
    for i in (1, 2):                                                       # the others are untouched
        assert res[i].token_ids == want[i] and seen_tokens[i] == want[i]
        assert res[i].text == texts[i] and seen_text[i] == texts[i] and res[i].stats.done_reason == "length"
    assert _all_free(eng)


def test_stop_strings_without_a_tokenizer_are_refused(tiny_dirs, cpu_ops):
    from hfee_b200 import Engine, SamplingOptions
    eng = Engine(tiny_dirs["A"], dtype="float32", page_size=16, max_requests=2, max_context=64, max_batch_tokens=32,
                 device="cpu")
    with pytest.raises(ValueError, match="tokenizer"):
        eng.generate([[1, 2, 3]], SamplingOptions.greedy(num_predict=2).with_(stop=["x"]))


@pytest.mark.parametrize("pipeline", [True, False])
def test_cancel_from_a_callback_and_through_the_cancel_set(tiny_dirs, cpu_ops, pipeline):
    """Request 1 is cancelled by its callback after three tokens, request 2 through the set while its
    prompt is still being read (small portions), request 3 before it was ever admitted (two slots);
    request 0 finishes with the plain implementation's tokens; every page and slot is free afterwards."""
    from hfee_b200 import SamplingOptions
    cfg, w = plain.load_model_dir(tiny_dirs["A"])
    rng = np.random.default_rng(22)
    prompts = [rng.integers(0, cfg.vocab, size=n).tolist() for n in (20, 25, 60, 9)]
    want = [plain.greedy_generate(cfg, w, p, 12) for p in prompts]
    eng = _engine(tiny_dirs, pipeline, max_requests=3, prefill_chunk=8)
    cancel = {3}
    seen = [[] for _ in prompts]

    def on_token(i, t):
        seen[i].append(t)
        if i == 0 and len(seen[0]) == 1:
            cancel.add(2)                      # request 2 (60 prompt tokens in portions of 8) is still reading
        return not (i == 1 and len(seen[1]) == 3)

    res = eng.generate(prompts, SamplingOptions.greedy(num_predict=12), on_token=on_token, cancel=cancel)
    assert res[0].token_ids == want[0] and res[0].stats.done_reason == "length"
    assert res[1].stats.done_reason == "abort" and res[1].token_ids == want[1][:len(res[1].token_ids)]
    assert 3 <= len(res[1].token_ids) <= 4 and seen[1] == res[1].token_ids[:len(seen[1])]
    assert res[2].stats.done_reason == "abort" and res[2].token_ids == []
    assert res[3].stats.done_reason == "abort" and res[3].token_ids == [] and res[3].stats.prompt_seconds == 0
    assert _all_free(eng)
    # the engine is usable afterwards
    again = eng.generate(prompts[:1], SamplingOptions.greedy(num_predict=12))
    assert again[0].token_ids == want[0]
