"""Token embedding (row gather, ullm/layers/vocab_parallel_embedding.py:117)
and the output head (ullm/layers/vocab_parallel_embedding.py:159-161).  No
vocabulary padding is kept: the kernels and the matrix product take any
vocabulary size.  A tied head reads the embedding table."""

from __future__ import annotations

from ..csrc import kernels
from .base import ParamDecl, Part


class TokenEmbedding(Part):
    """`scale` multiplies the gathered row; `position`, an encoding that `adds_to_embedding()`, is added to it;
    `param` is the table's name behind the part's prefix.  With either, or with a 32-bit stream under a 16-bit
    engine, `forward_stream` is the form to call: it writes the 32-bit stream and its rounded copy."""

    def __init__(self, vocab_size: int, hidden_size: int, scale: float = 1.0, position=None, param: str = "weight"):
        super().__init__()
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.scale = float(scale)
        self.position = position
        self.param = param

    def param_decls(self):
        return {self.param: ParamDecl((self.vocab_size, self.hidden_size))}

    @property
    def table(self):
        return self.tensors[self.param]

    def materialize(self, make):
        super().materialize(make)
        if self.position is not None:
            self.position.build_tables(self.table.device)

    def plain(self) -> bool:
        return self.scale == 1.0 and self.position is None

    def forward_stream(self, token_ids, stream, copy, ctx):
        """stream [T, hidden] float32 = table[id] * scale (+ the added position encoding); copy (the table's dtype,
        or None) = the rounded stream."""
        inv = self.position.tables()["inv_freq"] if self.position is not None else None
        kernels().embed_scaled(token_ids, self.table, stream, copy, self.scale, inv, ctx.positions if inv is not None else None,
                               ctx.last_tokens, ctx.token_req if ctx.last_tokens is not None else None,
                               ctx.req_slots if ctx.last_tokens is not None else None)
        return stream

    def forward(self, token_ids, out, ctx=None):
        """An id of -1 stands for the token its request sampled last, when the step's context carries the
        device array that holds those (`ctx.last_tokens`)."""
        if ctx is not None and ctx.last_tokens is not None:
            kernels().embedding(token_ids, self.table, out, ctx.last_tokens, ctx.token_req, ctx.req_slots)
        else:
            kernels().embedding(token_ids, self.table, out)
        return out


class TokenSideTable(Part):
    """A second table indexed by token id, [vocab, shares * dim]: share i (columns i * dim .. (i + 1) * dim) is what
    layer i reads of its tokens' rows.  The model puts the part into the step's context (`ctx.token_side`); a
    block that takes a per-layer token input reads `table` with its own share's offset."""

    def __init__(self, vocab_size: int, dim: int, shares: int, param: str = ""):
        super().__init__()
        if min(vocab_size, dim, shares) <= 0:
            raise ValueError("a token side table needs positive sizes")
        self.vocab_size, self.dim, self.shares, self.param = vocab_size, dim, shares, param

    def param_decls(self):
        return {self.param: ParamDecl((self.vocab_size, self.shares * self.dim))}

    @property
    def table(self):
        return self.tensors[self.param]


class OutputHead(Part):
    """logits = h W^T in 32-bit output, then optionally capped: cap * tanh(logits / cap).  `tied_to`, when set, is
    the embedding part whose table is read and no tensor of its own is declared."""

    def __init__(self, vocab_size: int, hidden_size: int, tied_to: TokenEmbedding | None = None, param: str = "weight",
                 softcap: float | None = None):
        super().__init__()
        if softcap is not None and not softcap > 0:
            raise ValueError("a logit cap must be positive")
        self.softcap = softcap
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.tied_to = tied_to
        self.param = param

    def param_decls(self):
        if self.tied_to is not None:
            return {}
        return {self.param: ParamDecl((self.vocab_size, self.hidden_size))}

    def weight(self):
        return self.tied_to.table if self.tied_to is not None else self.tensors[self.param]

    def forward(self, h, out_f32):
        kernels().linear_f32_out(h, self.weight(), out_f32)
        if self.softcap is not None:
            kernels().softcap_f32(out_f32, self.softcap)
        return out_f32
