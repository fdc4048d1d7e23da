"""Batched decoding of extraction slots right after the scoring pass that read them: the counterpart of spinf_serve/decode.py
(Group :23-36, GroupKV :53-68, Decoder :107-189 and its step :334-377, `_reorder` :322-329) on this library's kernels.

The scoring pass captured (GemmaStack.capture) the K/V of a tree's shared prefix and of every template branch. All slots of all
groups of a chunk then decode together, one token per slot and step: one row of the step's batch per (group, slot). A slot
attends to its group's prefix (stored once per group), to its own prompt's template and to the tokens its own beam generated
(ops.x_attention): nothing is copied per slot or beam. The step is the stack's ordinary layer chain (GemmaStack.forward) with that
attention in place of the tree attention, on static buffers, so it can be captured in a CUDA graph and replayed.

Tensors are token-major here ([groups, tokens, kv heads, dim]), the form the capture delivers, where the reference keeps
[groups, kv heads, tokens, dim]."""

from dataclasses import dataclass, field

import torch

from spinf_serve_b200 import ops

BEAM = 6  # live beams per prompt and step (extract.BEAM, spinf_serve/extract.py:33)
PAD_TOKEN = 0


@dataclass
class Group:
    """one tree's captured state: prefix K/V by layer ((k, v), each [stored tokens, kv heads, dim]; sliding layers the last
    window - 1 tokens), the prefix length P, and the prompts: (prompt, {layer: (k, v)} of its template, template length T, the
    final hidden state [hidden] at the template's last token, from which step 0 reads its log-probs: the reference keeps the
    [vocab] log-probs themselves there). A prompt needs `.key` and `.max_tokens`."""

    prefix_kv: dict
    P: int
    prompts: list = field(default_factory=list)
    extra: dict | None = None
    extra_bytes: int = 0


def _stored_prefix(g: Group, layer) -> int:
    """tokens of the group's prefix a layer keeps (a sliding layer's capture is already cut to its window)"""
    kv = g.prefix_kv.get(layer)
    return g.P if kv is None else kv[0].shape[0]


def _padded_bytes(per_tok_kv: dict, n_groups: int, prefix_of, template_tokens: int, slots: int, steps: int) -> int:
    """K/V bytes of a decoder holding, per layer, n_groups x (prefix + templates once, `steps` generated tokens per slot)"""
    return sum(per_tok * n_groups * (prefix_of(layer) + template_tokens + slots * steps) for layer, per_tok in per_tok_kv.items())


def group_bytes(g: Group, per_tok_kv: dict, S: int, beam: int = BEAM) -> int:
    """the decoder's memory for one group alone (the quantity decode.group_bytes estimates, spinf_serve/decode.py:392-402):
    per_tok_kv maps each layer with K/V to the bytes one token takes there; S generated tokens per slot"""
    templates = sum(p[2] for p in g.prompts)
    return g.extra_bytes + _padded_bytes(per_tok_kv, 1, lambda layer: _stored_prefix(g, layer), templates, len(g.prompts) * beam, S)


def chunk_bytes(groups: list, per_tok_kv: dict, extra: int = 0, beam: int = BEAM) -> int:
    """the decoder's memory for groups decoded together (decode.chunk_bytes, :378-391): Decoder pads every group to the chunk's
    longest prefix, largest template total, most prompts and largest token limit, so a chunk costs more than its groups' sum"""
    slots = beam * max(len(g.prompts) for g in groups)
    steps = 1 + max(p[0].max_tokens for g in groups for p in g.prompts)
    templates = max(sum(p[2] for p in g.prompts) for g in groups)
    return extra + _padded_bytes(per_tok_kv, len(groups), lambda layer: max(_stored_prefix(g, layer) for g in groups), templates, slots, steps)


class Decoder:
    """one chunk of groups decoded together"""

    def __init__(self, stack, groups: list, device, beam: int = BEAM, graphs: bool = False):
        self.stack, self.groups, self.device, self.beam, self.graphs = stack, groups, device, beam, graphs
        cfg = stack.cfg
        self.kv_layers = sorted(groups[0].prefix_kv)
        G = self.G = len(groups)
        J = max(len(g.prompts) for g in groups)
        Q = self.Q = J * beam
        S = self.S = max(p.max_tokens for g in groups for p, *_ in g.prompts) + 1
        h, D = cfg.kv_heads, cfg.head_dim
        Tt = self.Tt = max(sum(T for _, _, T, _ in g.prompts) for g in groups)
        pos_t = torch.full((G, Tt), -1, dtype=torch.int32)
        own_t = torch.full((G, Tt), -1, dtype=torch.int32)
        base = torch.zeros((G, Q), dtype=torch.int32)
        for gi, g in enumerate(groups):
            o = 0
            pos0 = g.extra.get("pos0") if g.extra else None
            for j, (_, _, T, _) in enumerate(g.prompts):
                pos_t[gi, o : o + T] = torch.arange(g.P, g.P + T, dtype=torch.int32)
                own_t[gi, o : o + T] = j
                base[gi, j * beam : (j + 1) * beam] = pos0[j] if pos0 else g.P + T
                o += T
        self.pos_t, self.own_t, self.base = pos_t.to(device), own_t.to(device), base.to(device)
        self.kp, self.vp, self.pos_p, self.kt, self.vt, self.gk, self.gv = {}, {}, {}, {}, {}, {}, {}
        bf = torch.bfloat16
        for li in self.kv_layers:
            Lp = max(g.prefix_kv[li][0].shape[0] for g in groups)
            kp, vp = torch.zeros((G, Lp, h, D), dtype=bf, device=device), torch.zeros((G, Lp, h, D), dtype=bf, device=device)
            pos = torch.full((G, Lp), -1, dtype=torch.int32)
            kt, vt = torch.zeros((G, Tt, h, D), dtype=bf, device=device), torch.zeros((G, Tt, h, D), dtype=bf, device=device)
            for gi, g in enumerate(groups):
                k, v = g.prefix_kv[li]
                n = k.shape[0]
                kp[gi, :n], vp[gi, :n] = k, v
                pos[gi, :n] = torch.arange(g.P - n, g.P, dtype=torch.int32)  # a sliding layer keeps the last n of the prefix
                o = 0
                for _, tkv, T, _ in g.prompts:
                    kt[gi, o : o + T], vt[gi, o : o + T] = tkv[li]
                    o += T
            self.kp[li], self.vp[li], self.pos_p[li], self.kt[li], self.vt[li] = kp, vp, pos.to(device), kt, vt
            self.gk[li] = torch.zeros((G, Q, S, h, D), dtype=bf, device=device)
            self.gv[li] = torch.zeros((G, Q, S, h, D), dtype=bf, device=device)
            for g in groups:  # the captured tensors are copied: let them go
                g.prefix_kv[li] = None
        for g in groups:
            for p in g.prompts:
                p[1].clear()
        # the static buffers of a step (a captured graph replays on them)
        self.qpos = self.base.clone()
        self.tok_buf = torch.full((G, Q), PAD_TOKEN, dtype=torch.int64, device=device)
        self.step_t = torch.zeros(1, dtype=torch.int64, device=device)
        self.step32 = torch.zeros(1, dtype=torch.int32, device=device)
        need = int(ops._lib.lib().spinf_x_attention_workspace_bytes(G, Q, cfg.heads, D, max(k.shape[1] for k in self.kp.values()), Tt, S))
        self.workspace = torch.empty(need, dtype=torch.uint8, device=device)
        self.step = 0
        self.graph, self.h_out = None, None
        self.scaling = 1.0  # the Gemma-style layers norm q and k and attend with scaling 1

    def _attend(self, i, kind, q, k, v):
        """a layer's attention inside a step: the new tokens' K/V into the generated range at the current step (GroupKV.update,
        done by the attention's first launch) and the three-range attention"""
        G, Q, S = self.G, self.Q, self.S
        cfg = self.stack.cfg
        h, D = cfg.kv_heads, cfg.head_dim
        window = cfg.window if kind == "sliding_attention" else None
        out = ops.x_attention(
            q.view(G, Q, cfg.heads, D), self.kp[i], self.vp[i], self.pos_p[i], self.kt[i], self.vt[i], self.pos_t, self.own_t, self.gk[i],
            self.gv[i], self.qpos, self.step32, self.beam, self.scaling, window, None, workspace=self.workspace, k_new=k, v_new=v,
        )
        return out.view(G * Q, cfg.heads, D)

    def _step_once(self):
        inputs = {"ids": self.tok_buf.reshape(1, -1), "pos": self.qpos.reshape(1, -1)}
        return self.stack.forward(None, None, inputs, None, attend=self._attend).reshape(self.G, self.Q, -1)

    def forward(self, tokens, step: int | None = None):
        """one decoding step: tokens [G, Q] int64 (PAD_TOKEN in unused slots) at step `step` (default: the next one) -> hidden
        states after the last norm [G, Q, hidden]. With graphs=True the step is captured once, after one run outside the capture,
        and replayed afterwards (Decoder._forward, decode.py:334-357)."""
        if step is not None:
            self.step = step
        self.tok_buf.copy_(tokens)
        self.qpos.copy_(self.base + self.step)
        self.step_t.fill_(self.step)
        self.step32.fill_(self.step)
        self._prepare(self.step)
        self.step += 1
        out = self._run()
        self._finish()
        return out

    def _prepare(self, step: int) -> None:
        """a family's own static buffers for this step (before the step runs, outside a captured graph)"""

    def _finish(self) -> None:
        """a family's bookkeeping after the step (outside a captured graph)"""

    def _run(self):
        if self.graph is not None:
            self.graph.replay()
            return self.h_out
        if not self.graphs:
            return self._step_once()
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            self._step_once()  # lazy initialisations must not happen inside the capture; the step is idempotent
        torch.cuda.current_stream(self.device).wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.h_out = self._step_once()
        self.graph = g
        g.replay()
        return self.h_out

    def reorder(self, parent) -> None:
        """the generated K/V follow their beams: slot s takes slot parent[s]'s (parent: int64 [G * Q] on the device), in place"""
        for li in self.kv_layers:
            for t in (self.gk[li], self.gv[li]):
                flat = t.view(self.G * self.Q, *t.shape[2:])
                flat.copy_(flat[parent])


class HybridDecoder(Decoder):
    """Decoder for the hybrid family (qwen_stack.QwenStack): the attention layers as above; a recurrent layer re-runs the gated
    delta rule from the group's prefix state over the slot's own rows (its template's, once per prompt for all its beams, then the tokens it generated): no per-slot
    state is kept or copied when beams fan out, only the small row caches follow the beams; the 4-tap convolution reads a
    per-slot ring of the three previous pre-convolution rows (spinf_serve/models/qwen35/qwen_decode.py:1-20,70-166). A group's
    `extra` holds what QwenStack.capture delivered for it: {"state": {layer: S}, "tmpl": [per prompt {"tok": {layer: (q, k, v, g,
    beta)}, "pre": {layer: [3, conv dim]}}]}."""

    def __init__(self, stack, groups: list, device, beam: int = BEAM, graphs: bool = False):
        extras = [g.extra for g in groups]
        for g in groups:
            g.extra = None  # the base class reads extra["pos0"] only
        super().__init__(stack, groups, device, beam, graphs)
        cfg = stack.cfg
        self.scaling = cfg.head_dim**-0.5
        G, Q, S = self.G, self.Q, self.S
        n = self.n = G * Q
        self.rec = [i for i in range(stack.n_layers) if stack.w.layers[i]["kind"] == "linear_attention"]
        self.rec_pos = {li: x for x, li in enumerate(self.rec)}
        n_g = len(self.rec)
        hk, hv, dk, dv = cfg.hk, cfg.hv, cfg.dk, cfg.dv
        cd = self.cd = 2 * hk * dk + hv * dv
        width = cd + hv * dv + 2 * hv  # an in-projection row: q | k | v | z | b | a
        bf = torch.bfloat16
        self.h0 = torch.empty((n_g, G, hv, dk, dv), dtype=torch.float32, device=device)
        for x, li in enumerate(self.rec):
            for gi, e in enumerate(extras):
                self.h0[x, gi].copy_(e["state"][li])
        self.h0_idx = (torch.arange(n, dtype=torch.int64) // Q).to(device)
        # row caches per recurrent layer: the templates' rows (prompt after prompt), then S generated rows per slot
        t0, r = {}, 0
        for gi, g in enumerate(groups):
            for j, (_, _, T, _) in enumerate(g.prompts):
                t0[(gi, j)] = r
                r += T
        self.gen0 = r
        R = self.R = r + n * S
        self.cq = torch.zeros((n_g, R, hk, dk), dtype=bf, device=device)
        self.ck = torch.zeros((n_g, R, hk, dk), dtype=bf, device=device)
        self.cv = torch.zeros((n_g, R, hv, dv), dtype=bf, device=device)
        self.cg = torch.zeros((n_g, R, hv), dtype=torch.float32, device=device)
        self.cb = torch.zeros((n_g, R, hv), dtype=bf, device=device)
        # in-projection rows of a step with the conv rings behind them: rows 0 .. n - 1 the step's own, rows n + 3 s .. n + 3 s + 2
        # slot s's three previous pre-convolution rows (taps 3 back .. 1 back); one prologue call reads both through its tap table
        self.ybuf = torch.zeros((n_g, 4 * n, width), dtype=bf, device=device)
        for gi, (g, e) in enumerate(zip(groups, extras, strict=True)):
            for j, (_, _, T, _) in enumerate(g.prompts):
                a = t0[(gi, j)]
                sl = slice(gi * Q + j * beam, gi * Q + (j + 1) * beam)
                for x, li in enumerate(self.rec):
                    q, k, v, gg, bb = e["tmpl"][j]["tok"][li]
                    self.cq[x, a : a + T], self.ck[x, a : a + T], self.cv[x, a : a + T] = q, k, v
                    self.cg[x, a : a + T], self.cb[x, a : a + T] = gg, bb
                    ring = self.ybuf[x, n:].view(n, 3, width)
                    ring[sl, :, :cd] = e["tmpl"][j]["pre"][li][None]
        s_ar = torch.arange(n, dtype=torch.int64)
        self.conv_idx = torch.stack([n + 3 * s_ar, n + 3 * s_ar + 1, n + 3 * s_ar + 2, s_ar], 1).contiguous().to(device)
        # The recurrence of a step runs as two calls. First every prompt's template rows from its group's prefix state (the beams of
        # a prompt share them: once per prompt, not once per slot), leaving the state at the template's end in `ht` (one buffer for
        # all layers: the second call of the same layer consumes it); a prompt slot without a prompt has no rows and passes the
        # prefix state on. Then every slot's generated rows 0 .. step from its prompt's entry of `ht`. The state goes through memory
        # in fp32 unchanged, so a slot sees the same sequence of updates as one call over template + generated rows would give it.
        J = Q // beam
        t_len = torch.zeros(G * J, dtype=torch.int64)
        for gi, g in enumerate(groups):
            for j, (_, _, T, _) in enumerate(g.prompts):
                t_len[gi * J + j] = T
        self.t_cu = torch.nn.functional.pad(t_len.cumsum(0), (1, 0)).contiguous().to(device)  # rows 0 .. gen0 - 1, prompt after prompt
        self.t_h0_idx = (torch.arange(G * J, dtype=torch.int64) // J).to(device)
        self.t_ht_idx = torch.arange(G * J, dtype=torch.int64, device=device)
        self.ht = torch.empty((G * J, hv, dk, dv), dtype=torch.float32, device=device)
        self.slot_prompt = (s_ar // beam).to(device)
        # the generated rows of every step, made once on the host: slot s, step st -> rows gen0 + s S + (0 .. st)
        steps = torch.arange(1, S + 1, dtype=torch.int64)
        self.cu_all = (steps[:, None] * torch.arange(n + 1, dtype=torch.int64)[None, :]).contiguous().to(device)  # [S, n + 1]
        idx_all = torch.zeros((S, n * S), dtype=torch.int64)
        for st in range(S):
            idx_all[st, : n * (st + 1)] = (self.gen0 + s_ar[:, None] * S + torch.arange(st + 1)[None, :]).reshape(-1)
        self.idx_all = idx_all.to(device)
        self.gen_row0 = (self.gen0 + s_ar * S).to(device)
        # static buffers of a step
        self.idx_buf = self.idx_all[0].clone()
        self.cu_buf = self.cu_all[0].clone()
        self.cur_rows = self.gen_row0.clone()
        self.o_buf = torch.zeros((R, hv, dv), dtype=bf, device=device)

    def _prepare(self, step: int) -> None:
        st = min(step, self.S - 1)
        self.idx_buf.copy_(self.idx_all[st])
        self.cu_buf.copy_(self.cu_all[st])
        self.cur_rows.copy_(self.gen_row0 + st)

    def _finish(self) -> None:
        """the conv rings advance by the step's own pre-convolution rows"""
        n, cd = self.n, self.cd
        ring = self.ybuf[:, n:].view(len(self.rec), n, 3, -1)
        ring[:, :, 0, :cd] = ring[:, :, 1, :cd].clone()
        ring[:, :, 1, :cd] = ring[:, :, 2, :cd].clone()
        ring[:, :, 2, :cd] = self.ybuf[:, :n, :cd]

    def _attend_q(self, i, q, k, v):
        G, Q = self.G, self.Q
        cfg = self.stack.cfg
        h, D = cfg.kv_heads, cfg.head_dim
        out = ops.x_attention(
            q.view(G, Q, cfg.heads, D), self.kp[i], self.vp[i], self.pos_p[i], self.kt[i], self.vt[i], self.pos_t, self.own_t, self.gk[i],
            self.gv[i], self.qpos, self.step32, self.beam, self.scaling, None, None, workspace=self.workspace, k_new=k, v_new=v,
        )
        return out.view(G * Q, cfg.heads, D)

    def _recur(self, i, y):
        """a recurrent layer inside a step: the step's in-projection rows next to the rings, the fused steps before the recurrence
        through the tap table, the new rows into the caches, the recurrence from the prefix state over every slot's rows; the
        outputs of the step's own rows come back"""
        from spinf_serve_b200 import gdn

        cfg, L = self.stack.cfg, self.stack.w.layers[i]
        x, n = self.rec_pos[i], self.n
        yb = self.ybuf[x]
        yb[:n].copy_(y)
        q, k, v, z, g, beta = gdn.prologue(yb, self.conv_idx, L["conv_w"], L["A_log"], L["dt_bias"], cfg.hk, cfg.dk, cfg.hv, cfg.dv, n_tokens=n)
        self.cq[x].index_copy_(0, self.cur_rows, q)
        self.ck[x].index_copy_(0, self.cur_rows, k)
        self.cv[x].index_copy_(0, self.cur_rows, v)
        self.cg[x].index_copy_(0, self.cur_rows, g)
        self.cb[x].index_copy_(0, self.cur_rows, beta)
        rows = (self.cq[x], self.ck[x], self.cv[x], self.cg[x], self.cb[x])
        if self.gen0:
            gdn.recurrent(*rows, cfg.dk**-0.5, self.t_cu, self.t_cu.numel() - 1, h0=self.h0[x], h0_idx=self.t_h0_idx, ht=self.ht,
                          ht_idx=self.t_ht_idx, o=self.o_buf)
            gdn.recurrent(*rows, cfg.dk**-0.5, self.cu_buf, n, h0=self.ht, h0_idx=self.slot_prompt, idx=self.idx_buf, o=self.o_buf)
        else:  # no prompt has template tokens: the slots start from their groups' prefix states
            gdn.recurrent(*rows, cfg.dk**-0.5, self.cu_buf, n, h0=self.h0[x], h0_idx=self.h0_idx, idx=self.idx_buf, o=self.o_buf)
        return self.o_buf.index_select(0, self.cur_rows), z

    def _step_once(self):
        inputs = {"ids": self.tok_buf.reshape(1, -1), "pos": self.qpos.reshape(1, -1)}
        return self.stack.forward(None, None, inputs, None, attend=self._attend_q, recur=self._recur).reshape(self.G, self.Q, -1)

    def reorder(self, parent) -> None:
        """as Decoder.reorder, plus the generated rows of the recurrent caches and the conv rings (qwen_decode.Decoder._reorder)"""
        super().reorder(parent)
        n, S = self.n, self.S
        for t in (self.cq, self.ck, self.cv, self.cg, self.cb):
            for x in range(t.shape[0]):  # layer by layer: the gather's temporary is one layer's rows
                gen = t[x, self.gen0 :].view(n, S, *t.shape[2:])
                gen.copy_(gen[parent])
        ring = self.ybuf[:, n:].view(len(self.rec), n, 3, -1)
        ring.copy_(ring[:, parent])


def search_text(dec: Decoder, lm_weight, stop_ids, banned_ids=(), topk: int | None = None, min_p: float = 0.002, softcap=None):
    """beam search over every prompt of the decoder's groups at once, the text kind of Decoder.run (decode.py:191-320 with
    extract.py's constants): a beam ends with the summed probability of the stop tokens; the `topk` best continuations of every
    live beam compete for the prompt's `beam` slots; beams below min_p are dropped. -> {prompt key: [(tokens, log-prob)] best
    first}. Candidates are picked from bf16 logits (twice as many as needed) and ranked by their exact fp32 log-probs."""
    import math

    beam = dec.beam
    topk = topk or beam
    G, Q = dec.G, dec.Q
    dev = dec.device
    stop = torch.as_tensor(sorted(stop_ids), dtype=torch.int64, device=dev)
    mask_ids = torch.as_tensor(sorted(set(stop_ids) | set(banned_ids)), dtype=torch.int64, device=dev)
    prompts = [(gi, j, p) for gi, g in enumerate(dec.groups) for j, (p, *_) in enumerate(g.prompts)]
    found = {p.key: [] for _, _, p in prompts}
    live = {p.key: [(0.0, [])] for _, _, p in prompts}
    slots = {p.key: [gi * Q + j * beam] for gi, j, p in prompts}
    floor = math.log(min_p)

    def read(h_rows):
        """h_rows [R, hidden] -> (end log-prob [R], candidate ids [R, 2 topk], their log-probs)"""
        logits = ops.bf16_gemm(h_rows, lm_weight).float()
        logits[:, mask_ids] = -float("inf")
        cand = logits.topk(2 * topk, -1).indices
        cols = torch.unique(torch.cat([cand.reshape(-1), stop]))
        lp = ops.option_logprobs(h_rows, lm_weight, cols.to(torch.int32), softcap)
        end = torch.logsumexp(lp[:, torch.searchsorted(cols, stop)], -1)
        return end.cpu().numpy(), cand.cpu().numpy(), torch.gather(lp, 1, torch.searchsorted(cols, cand)).cpu().numpy()

    # step 0 reads the scoring pass's hidden state at the end of each template: the caller put it in the prompt tuple as the 4th item
    h0 = torch.stack([dec.groups[gi].prompts[j][3] for gi, j, _ in prompts])
    end, cand, clp = read(h0)
    row_of = {gi * Q + j * beam: k for k, (gi, j, _) in enumerate(prompts)}
    for step in range(dec.S):
        tokens = torch.full((G * Q,), PAD_TOKEN, dtype=torch.int64)
        parent = torch.arange(G * Q)
        new_slots = {}
        for gi, j, p in prompts:
            beams, old = live[p.key], slots[p.key]
            if not beams:
                continue
            pool = []
            for b, (s, toks) in enumerate(beams):
                r = row_of[old[b]]
                if toks:
                    found[p.key].append((toks, s + float(end[r])))
                order = sorted(range(cand.shape[1]), key=lambda t: -clp[r, t])[:topk]
                pool += [(s + float(clp[r, t]), b, int(cand[r, t])) for t in order]
            if step >= p.max_tokens:
                live[p.key], new_slots[p.key] = [], []
                continue
            best = max((x[1] for x in found[p.key]), default=-float("inf"))
            pool = [c for c in sorted(pool, key=lambda c: -c[0]) if c[0] >= max(floor, best + math.log(0.02))][:beam]
            live[p.key] = [(c[0], beams[c[1]][1] + [c[2]]) for c in pool]
            new_slots[p.key] = [gi * Q + j * beam + b for b in range(len(pool))]
            for sl, c in zip(new_slots[p.key], pool, strict=True):
                parent[sl] = old[c[1]]
                tokens[sl] = c[2]
        slots = {k: new_slots.get(k, []) for k in slots}
        alive = sorted(s for v in slots.values() for s in v)
        if not alive:
            break
        if step > 0 and not bool((parent == torch.arange(G * Q)).all()):
            dec.reorder(parent.to(dev))
        h = dec.forward(tokens.view(G, Q).to(dev), step)
        row_of = {s: k for k, s in enumerate(alive)}
        end, cand, clp = read(h.reshape(G * Q, -1)[torch.as_tensor(alive, device=dev)].contiguous())
    return {k: sorted(v, key=lambda x: -x[1]) for k, v in found.items()}
