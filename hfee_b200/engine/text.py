"""Text of a request as it is generated: whole UTF-8 characters only, and nothing that
may turn out to be the start of a stop string.

The two small state machines of hostfog/hfee internal/llm/text.go: ``Utf8Buffer``
(text.go:16-39) holds bytes back until they form complete characters, since one
character can be split over tokens; ``Stopper`` (text.go:41-78) withholds text that
could begin a stop string and reports a hit without ever giving the stop string
out.  ``TextStream`` joins them per request the way ``Runner.sample`` does
(runner.go:283-312): piece of the token -> characters -> leading spaces of the
answer dropped -> stopper -> released text; it also remembers where each token's
text ended, so that the tokens wholly in front of a stop string can be told from
the ones it cut.
"""
from __future__ import annotations

from typing import Any, List, Optional, Sequence, Tuple

_UTF_MAX = 4


class Utf8Buffer:
    """Bytes in, complete characters out (text.go:16-39)."""

    def __init__(self) -> None:
        self.pending = b""

    def add(self, piece: bytes) -> str:
        self.pending += piece
        for cut in range(0, min(_UTF_MAX, len(self.pending)) + 1):
            end = len(self.pending) - cut
            try:
                out = self.pending[:end].decode("utf-8")
            except UnicodeDecodeError:
                continue
            self.pending = self.pending[end:]
            return out
        return self.flush()

    def flush(self) -> str:
        out = self.pending.decode("utf-8", errors="replace")
        self.pending = b""
        return out


class Stopper:
    """Withholds text that might be the start of a stop string (text.go:41-78)."""

    def __init__(self, stops: Sequence[str]):
        self.stops = [s for s in stops if s]
        self.buf = ""

    def push(self, text: str) -> Tuple[str, bool]:
        """Add ``text``; returns (text that may be given out now, whether a stop string was
        found).  On a hit the text in front of the stop string is returned and the rest dropped."""
        self.buf += text
        for stop in self.stops:
            i = self.buf.find(stop)
            if i >= 0:
                out, self.buf = self.buf[:i], ""
                return out, True
        hold = 0
        for stop in self.stops:
            for k in range(min(len(stop) - 1, len(self.buf)), hold, -1):
                if self.buf.endswith(stop[:k]):
                    hold = k
                    break
        cut = len(self.buf) - hold
        out, self.buf = self.buf[:cut], self.buf[cut:]
        return out, False

    def flush(self) -> str:
        out, self.buf = self.buf, ""
        return out


class TokenizerAdapter:
    """What the engine needs of a tokenizer, over either a ``tokenizers.Tokenizer`` or any
    object with ``encode(text)`` (a list of ids, or something with ``.ids``) and ``decode(ids)``;
    an object that also has ``piece(id) -> bytes`` (the reference's ``Tokenizer.Piece``) gives
    the bytes of single tokens directly."""

    def __init__(self, tok: Any):
        self.tok = tok
        self.has_piece = hasattr(tok, "piece")

    def encode(self, text: str) -> List[int]:
        try:
            enc = self.tok.encode(text, add_special_tokens=False)
        except TypeError:
            enc = self.tok.encode(text)
        return list(getattr(enc, "ids", enc))

    def decode(self, ids: Sequence[int]) -> str:
        return self.tok.decode(list(ids))

    def piece(self, token: int) -> bytes:
        return bytes(self.tok.piece(int(token)))


class TextStream:
    """One request's tokens -> the text that may be shown.

    ``push(token)`` returns (released text, stop string found).  After a hit, or at the end of
    the request, ``finish()`` returns what was still held back (nothing after a hit).
    ``whole_tokens`` is the number of leading tokens all of whose text has been released; after
    a hit those are the tokens in front of the stop string."""

    def __init__(self, tokenizer: TokenizerAdapter, stops: Sequence[str] = ()):
        self.tokenizer = tokenizer
        self.stopper = Stopper(stops)
        self.chars = Utf8Buffer()
        self.started = False
        self.hit = False
        self.text = ""                 # everything released so far
        self._ids: List[int] = []      # incremental decoding without single-token pieces
        self._prefix = 0
        self._read = 0
        self._fed = 0                  # characters given to the stopper so far
        self._ends: List[int] = []     # per token: characters given to the stopper once its text was in

    # ------------------------------------------------------------------ token -> characters
    def _characters(self, token: int) -> str:
        if self.tokenizer.has_piece:
            return self.chars.add(self.tokenizer.piece(token))
        # Decode a window of recent tokens with and without the new one; what the new one added is
        # the difference, unless it ends inside a character (the decoder then shows U+FFFD).
        self._ids.append(int(token))
        before = self.tokenizer.decode(self._ids[self._prefix:self._read])
        now = self.tokenizer.decode(self._ids[self._prefix:])
        if len(now) > len(before) and not now.endswith("�"):
            self._prefix, self._read = self._read, len(self._ids)
            return now[len(before):]
        return ""

    def _rest_of_characters(self) -> str:
        if self.tokenizer.has_piece:
            return self.chars.flush()
        before = self.tokenizer.decode(self._ids[self._prefix:self._read])
        now = self.tokenizer.decode(self._ids[self._prefix:])
        self._prefix = self._read = len(self._ids)
        return now[len(before):]

    # ------------------------------------------------------------------ the stream
    def push(self, token: int) -> Tuple[str, bool]:
        if self.hit:
            return "", True
        text = self._characters(token)
        if not self.started:                       # runner.go:298-301: the answer starts at its first non-space
            text = text.lstrip(" ")
            self.started = text != ""
        self._fed += len(text)
        self._ends.append(self._fed)
        out, self.hit = self.stopper.push(text)
        self.text += out
        return out, self.hit

    def finish(self) -> str:
        """What is still held back when the request ends without a stop string (runner.go:316-318)."""
        if self.hit:
            return ""
        rest = self._rest_of_characters()
        if not self.started:
            rest = rest.lstrip(" ")
        out = ""
        if rest:
            self._fed += len(rest)
            if self._ends:
                self._ends[-1] = self._fed
            out, self.hit = self.stopper.push(rest)
        if not self.hit:
            out += self.stopper.flush()
        self.text += out
        return out

    @property
    def whole_tokens(self) -> int:
        """Leading tokens whose text lies wholly inside what has been released."""
        n = 0
        for end in self._ends:
            if end > len(self.text):
                break
            n += 1
        return n
