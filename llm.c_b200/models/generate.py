"""Batched text generation with a key / value cache for the LLaMA family.

Capability parity with ``LLaMA.generate`` and ``sample_top_p`` of the reference script (train_llama3.py:476-576) and with the
cache inside its attention module (train_llama3.py:156-180): prompts of different lengths are decoded side by side, the prompt
part of every row is forced, each step runs only the tokens that are new since the previous step through the network, and
sampling is nucleus (top-p) at a temperature, or greedy at temperature 0.

The decoder works on the parameter tensors of a ``models.llama3.Llama`` (it never copies them), with its own small activation
set and the caches ``(L, max_batch, max_len, NKV, HS)``.  On a GPU every step is a chain of this library's kernels: the GEMMs
of training for prompts (rows padded to one 128-row tile) or a weight-streaming product for steps of at most 8 rows, RMSNorm / SwiGLU, and the two decoding kernels of csrc/decode.cu (rotary
embedding written straight into the cache; attention of the new queries over the cached keys with grouped heads read in
place).  A one-token step issues about nine small launches per layer and is bound by launch latency, so on a GPU it is
captured once in a CUDA graph and replayed (``GraphStep``): the position lives in device memory, the graph advances it itself,
and the kernels refuse a position outside the cache through the library's status word.  On the CPU the same chain runs on
the fp32 restatement of the operators.
"""
import torch

from .. import ops


class CachedDecoder:
    def __init__(self, model, max_batch, max_len):
        cfg = model.cfg
        if max_len > cfg.max_seq_len:
            raise ValueError("cache length %d exceeds the model's context %d" % (max_len, cfg.max_seq_len))
        self.model = model
        self.max_batch, self.max_len = max_batch, max_len
        L, NKV, HS = cfg.num_layers, cfg.num_kv_heads, cfg.head_size
        self.kcache = torch.zeros(L, max_batch, max_len, NKV, HS, dtype=model.dtype, device=model.device)
        self.vcache = torch.zeros_like(self.kcache)
        self._rows = 0
        self._bufs = None
        self._dense = None
        # prompts of at least this many tokens per row, starting at position 0, run through the training attention kernel
        self.dense_prefill_from = 128
        # steps of at most this many rows use the weight-streaming product instead of a padded tensor-core tile (0: never)
        self.skinny_rows = 8 if (model.device.type == "cuda" and model.dtype == torch.bfloat16) else 0

    def cache_bytes(self):
        return 2 * self.kcache.numel() * self.kcache.element_size()

    def _buffers(self, N, B):
        """Activation rows are padded to a multiple of 128 so that every product is made of whole tiles; the rows beyond N
        stay zero and are never read back."""
        rows = (max(N, B) + 127) // 128 * 128
        if rows > self._rows:
            m, cfg = self.model, self.model.cfg
            C, H, Vp = cfg.channels, cfg.hidden_dim, cfg.padded_vocab_size
            QR = (cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_size
            z = lambda *s, dtype=m.dtype: torch.zeros(*s, dtype=dtype, device=m.device)
            self._bufs = dict(x=z(rows, C), ln=z(rows, C), rstd=z(rows, dtype=torch.float32), raw=z(rows, QR), q=z(rows, C), atty=z(rows, C),
                              proj=z(rows, C), res=z(rows, C), fc12=z(rows, 2 * H), h=z(rows, H), last=z(128 * ((B + 127) // 128), C),
                              logits=z(128 * ((B + 127) // 128), Vp))
            self._rows = rows
        return self._bufs, rows

    def forward(self, tokens, start_pos, pos=None):
        """tokens (B, Tq) int32 on the model's device: the tokens at positions start_pos .. start_pos + Tq - 1 of every row.
        Returns the fp32 logits (B, vocab_size) of the last of them; keys and values of all of them enter the cache.
        With ``pos`` (one int32 on the device) the position is read by the kernels when they run and start_pos is ignored."""
        m = self.model
        cfg, p = m.cfg, m.params
        B, Tq = tokens.shape
        if B > self.max_batch or (pos is None and start_pos + Tq > self.max_len):
            raise ValueError("batch %d / positions up to %d exceed the cache (%d, %d)" % (B, start_pos + Tq, self.max_batch, self.max_len))
        if m.param_sync is not None and pos is None:
            m.param_sync.wait_all()            # (a replayed step follows a prefill that has waited already)
        N = B * Tq
        a, rows = self._buffers(N, B)
        L, NH, NKV, eps, C = cfg.num_layers, cfg.num_heads, cfg.num_kv_heads, cfg.norm_eps, cfg.channels
        x, ln, rstd = a["x"], a["ln"], a["rstd"]
        padded = m.device.type == "cuda"

        def mm(out, inp, weight, n):
            if n <= self.skinny_rows:
                ops.matmul_skinny(out[:n], inp[:n], weight)
            elif padded:
                ops.matmul_forward(out, inp, weight, None)          # whole 128-row tiles; the rows beyond n are never read
            else:
                ops.matmul_forward(out[:n], inp[:n], weight, None)

        ops.encoder_forward(x[:N].view(B, Tq, C), tokens, p["wte"], None)
        ops.rmsnorm_forward(ln[:N], rstd[:N], x[:N], p["ln1w"][0], eps)
        # a long prompt from position 0 is the training forward pass: its attention kernel (tensor cores, one pass over the
        # keys per 128 queries) replaces the per-query scan of the cache, and keys / values are copied into the cache afterwards
        dense = pos is None and start_pos == 0 and Tq >= self.dense_prefill_from
        if dense:
            rep, HS = NH // NKV, cfg.head_size
            if self._dense is None or self._dense[0].shape[0] < N or self._dense[1].numel() < B * NH * Tq:
                self._dense = (torch.zeros(rows, 3 * C, dtype=m.dtype, device=m.device),
                               torch.zeros(B * NH * Tq, dtype=torch.float32, device=m.device))
            packed, lse = self._dense[0][:N], self._dense[1][:B * NH * Tq].view(B, NH, Tq)
        for l in range(L):
            mm(a["raw"], ln, p["qkvw"][l], N)
            if dense:
                ops.rope_forward(packed, a["raw"][:N], m.freqs, Tq, NH, NKV)
                ops.attention_forward(a["atty"][:N], lse, packed, B, Tq, NH)
                kv = packed.view(B, Tq, 3, NKV, rep, HS)
                self.kcache[l][:B, :Tq].copy_(kv[:, :, 1, :, 0])
                self.vcache[l][:B, :Tq].copy_(kv[:, :, 2, :, 0])
            else:
                ops.rope_cache(a["q"][:N], self.kcache[l], self.vcache[l], a["raw"][:N], m.freqs, Tq, start_pos, NH, NKV, pos)
                ops.cached_attention(a["atty"][:N], a["q"][:N], self.kcache[l], self.vcache[l], Tq, start_pos, NH, NKV, pos)
            mm(a["proj"], a["atty"], p["attprojw"][l], N)
            ops.rmsnorm_fused_residual_forward(a["res"][:N], ln[:N], rstd[:N], x[:N], a["proj"][:N], p["ln2w"][l], eps)
            mm(a["fc12"], ln, p["fc12w"][l], N)
            ops.swiglu_forward(a["h"][:N], a["fc12"][:N])
            mm(a["proj"], a["h"], p["fcprojw"][l], N)
            w = p["ln1w"][l + 1] if l + 1 < L else p["lnfw"]
            ops.rmsnorm_fused_residual_forward(x[:N], ln[:N], rstd[:N], a["res"][:N], a["proj"][:N], w, eps)
        a["last"][:B].copy_(ln[:N].view(B, Tq, C)[:, -1])
        mm(a["logits"], a["last"], p["lmhead"], B)
        return a["logits"][:B, :cfg.vocab_size].float()


class GraphStep:
    """The one-token step of a ``CachedDecoder`` for a fixed batch size, captured in a CUDA graph.  ``step(tokens)`` copies the
    (B, 1) tokens into the graph's input, replays it and returns the graph's logits tensor (B, vocab_size), which the next
    replay overwrites.  The graph ends by adding 1 to the device-resident position."""

    def __init__(self, decoder, batch, start_pos):
        dev = decoder.model.device
        self.decoder = decoder
        self.tokens = torch.zeros(batch, 1, dtype=torch.int32, device=dev)
        self.pos = torch.full((1,), start_pos, dtype=torch.int32, device=dev)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            decoder.forward(self.tokens, 0, pos=self.pos)      # buffers, tensor maps and kernel attributes exist before the capture;
        torch.cuda.current_stream(dev).wait_stream(side)       # what it wrote at start_pos is overwritten by the first real step
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.logits = decoder.forward(self.tokens, 0, pos=self.pos)
            self.pos.add_(1)

    def step(self, tokens):
        self.tokens.copy_(tokens.view_as(self.tokens), non_blocking=True)
        self.graph.replay()
        return self.logits


def sample_top_p(probs, top_p, generator=None):
    """Nucleus sampling: the smallest set of most likely tokens whose mass exceeds ``top_p`` is renormalised and sampled
    (reference: sample_top_p, train_llama3.py:559-576).  probs (B, V) -> token ids (B,)."""
    sorted_p, order = torch.sort(probs, dim=-1, descending=True)
    before = torch.cumsum(sorted_p, dim=-1) - sorted_p
    kept = torch.where(before > top_p, torch.zeros_like(sorted_p), sorted_p)
    kept = kept / kept.sum(dim=-1, keepdim=True)
    pick = torch.multinomial(kept, 1, generator=generator)
    return torch.gather(order, -1, pick).view(-1)


def generate(model, prompt_tokens, max_gen_len, temperature=0.6, top_p=0.9, echo=False, stop_tokens=(), pad_id=-1,
             generator=None, use_kv=True, decoder=None, use_graph=None):
    """prompt_tokens: list of token-id lists.  Returns the list of generated id lists (with the prompt in front if ``echo``),
    each cut at its first stop token.  ``use_kv=False`` recomputes the whole prefix at every step through the same decoder
    (the slow path the cache replaces; it exists to check the cache against).  ``use_graph`` (default: on for a CUDA model)
    replays the one-token steps from a CUDA graph."""
    cfg = model.cfg
    bsz = len(prompt_tokens)
    lens = [len(t) for t in prompt_tokens]
    if bsz == 0 or min(lens) == 0:
        raise ValueError("every prompt needs at least one token")
    if max(lens) > cfg.max_seq_len:
        raise ValueError("prompt of %d tokens exceeds the context of %d" % (max(lens), cfg.max_seq_len))
    total_len = min(cfg.max_seq_len, max_gen_len + max(lens))
    if decoder is None:
        decoder = CachedDecoder(model, bsz, total_len)
    dev = model.device
    if use_graph is None:
        use_graph = dev.type == "cuda"
    use_graph = bool(use_graph) and use_kv and dev.type == "cuda"
    graph_step = None
    tokens = torch.full((bsz, total_len), pad_id, dtype=torch.int64)
    for i, t in enumerate(prompt_tokens):
        tokens[i, :len(t)] = torch.tensor(t, dtype=torch.int64)
    given = tokens != pad_id
    stops = torch.tensor(sorted(stop_tokens), dtype=torch.int64)
    done = torch.zeros(bsz, dtype=torch.bool)
    prev = 0
    for cur in range(min(lens), total_len):
        lo = prev if use_kv else 0
        step_in = tokens[:, lo:cur].clamp(min=0).to(torch.int32).to(dev)      # positions below cur are always filled
        if use_graph and lo > 0 and cur - lo == 1:
            if graph_step is None:
                graph_step = GraphStep(decoder, bsz, lo)
            logits = graph_step.step(step_in).cpu()
            if int(graph_step.pos.item()) != cur:
                raise RuntimeError("decoding graph is at position %d, expected %d" % (int(graph_step.pos.item()), cur))
        else:
            logits = decoder.forward(step_in, lo).cpu()
        if temperature > 0:
            nxt = sample_top_p(torch.softmax(logits / temperature, dim=-1), top_p, generator)
        else:
            nxt = torch.argmax(logits, dim=-1)
        nxt = torch.where(given[:, cur], tokens[:, cur], nxt)
        tokens[:, cur] = nxt
        if stops.numel():
            done |= ~given[:, cur] & torch.isin(nxt, stops)
        prev = cur
        if bool(done.all()):
            break
    out = []
    for i, row in enumerate(tokens.tolist()):
        row = row[(0 if echo else lens[i]):lens[i] + max_gen_len]
        for s in stop_tokens:
            if s in row:
                row = row[:row.index(s)]
        out.append([t for t in row if t != pad_id])
    return out
