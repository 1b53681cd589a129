"""Decode-only GPT-2 tokenizer reading ``gpt2_tokenizer.bin`` (reference: llmc/tokenizer.h, train_gpt2.py:509-524)."""
import ctypes
import struct

from . import _hostlib


def write_tokenizer(path, token_bytes, eot):
    """token_bytes: list of bytes objects, one per token id (version-2 file)."""
    header = [0] * 256
    header[0], header[1], header[2], header[3] = 20240328, 2, len(token_bytes), eot
    with open(path, "wb") as f:
        f.write(struct.pack("<256I", *header))
        for b in token_bytes:
            assert len(b) <= 255
            f.write(struct.pack("<B", len(b)))
            f.write(b)


class Tokenizer:
    def __init__(self, path):
        self._lib = _hostlib.lib()
        self._h = None
        self.init_ok = False
        try:
            self._h = self._lib.llmc_tokenizer_new(path.encode())
        except Exception:
            self._h = None
        if self._h:
            self.init_ok = True
            self.vocab_size = self._lib.llmc_tokenizer_vocab(self._h)
            self.eot_token = self._lib.llmc_tokenizer_eot(self._h)
        else:
            self.vocab_size, self.eot_token = 0, 50256

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.llmc_tokenizer_free(self._h)
            self._h = None

    def decode(self, token):
        """Raw bytes of one token (None if the tokenizer is not loaded or the id is out of range)."""
        if not self.init_ok:
            return None
        buf = ctypes.create_string_buffer(256)
        n = self._lib.llmc_tokenizer_decode(self._h, int(token), buf, 256)
        return None if n < 0 else buf.raw[:n]


def printable(piece):
    """Text that is safe to print for a decoded piece: single-byte pieces are shown only if printable or whitespace."""
    if piece is None or len(piece) == 0:
        return ""
    if len(piece) == 1:
        c = piece[0]
        if not (32 <= c < 127 or c in (9, 10, 13)):
            return ""
    return piece.decode("utf-8", "replace")
