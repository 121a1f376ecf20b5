"""Step-wise serving engine: requests that come and go, prompts fed in portions, decoded tokens one by one, several
requests per step.

``Engine.step(entries, end)`` is the one step function: every entry brings the next tokens of a request (a whole prompt,
a portion of one, or a single decoded token) and the places among them whose logits are wanted; the engine gives a new
request a slot of the model's per-sequence state (seq_state.SlotState), lays the entries' tokens out as the rows of one
batch, cuts what exceeds the row budget into further passes, runs the model's ``forward_rows`` and frees the slots of the
requests named in ``end``.  ``Engine.generate`` is greedy decoding on top of it (argmax on the device); the trace runner
(bin/trace_run) drives the same ``step``.

A pass in which every request brings ONE token (a decode step) is launch-bound when run eagerly -- some sixty kernels of
a few microseconds each -- so it is captured as a CUDA graph the second time its shape comes up and replayed from then
on: the ids, portions and positions live in one static device buffer that the pinned copy refreshes before every replay;
the kernels read slots and positions from it, so one graph serves every step of that shape.  "Shape" is the number of
rows, whether logits are wanted, and the model's ``graph_class(longest history)``: whatever else its launches depend on
(Davasun: how many key ranges the attention splits a history into, ``ops.latent_attn_splits``; Bebulorn: nothing).  The graph replays the very kernels of the eager pass;
results are bit-identical.

The reference serves one static batch per generate() call (greedy_search.py:37-460); this is the request-level face the
step-wise models need.
"""
import numpy as np
import torch

from . import graphs, ops
from .seq_layers import StepBatch


class _StepGraph:
    """One captured decode pass: the static input buffer, the graph and the logits it writes."""

    def __init__(self, words, device):
        self.inputs = torch.zeros(max(words, 2), dtype=torch.int32, device=device)
        self.graph = None
        self.logits = None


class Engine:
    def __init__(self, model, max_tokens, max_requests=4, max_rows=4096, graphs=True):
        self.model = model
        self.max_rows = int(max_rows)
        self.graphs = bool(graphs) and model.device.type == "cuda"     # decode passes as CUDA graphs (module docstring)
        self._step_graphs = {}
        self.slots = model.new_state(int(max_requests), int(max_tokens))
        self.device = model.device
        self._host = self._copied = None

    # ---- batch assembly: one pinned staging buffer, one H2D copy per pass
    def _upload(self, ids, segs, meta, want, static=None):
        n_ids, n_seg, n_meta, n_want = len(ids), len(segs) * 4, len(meta) * 2, len(want)
        words = 2 * n_ids + n_seg + n_meta + n_want
        if self._host is None or self._host.numel() < words:
            self._host = torch.empty(max(2 * words, 1024), dtype=torch.int32)
            if self.device.type == "cuda":
                self._host = self._host.pin_memory()
                self._copied = torch.cuda.Event()
        elif self._copied is not None:
            self._copied.synchronize()                     # the previous pass's copy has left the staging buffer
        host = self._host[:max(words, 2)]
        a = host.numpy()
        a[:2 * n_ids].view(np.int64)[:] = np.asarray(ids, dtype=np.int64)
        o = 2 * n_ids
        a[o:o + n_seg] = np.asarray(segs, dtype=np.int32).reshape(-1)
        a[o + n_seg:o + n_seg + n_meta] = np.asarray(meta, dtype=np.int32).reshape(-1)
        if n_want:
            a[o + n_seg + n_meta:words] = np.asarray(want, dtype=np.int32)
        if static is not None:
            dev = static[:host.numel()]
            dev.copy_(host, non_blocking=True)
        else:
            dev = host.to(self.device, non_blocking=True)
        if self._copied is not None:
            self._copied.record()
        elif dev.data_ptr() == host.data_ptr():
            dev = dev.clone()                              # host-resident models (tests): do not alias the staging buffer
        d_ids = dev[:2 * n_ids].view(torch.int64)
        d_segs = dev[o:o + n_seg].view(-1, 4)
        d_meta = dev[o + n_seg:o + n_seg + n_meta].view(-1, 2)
        d_want = dev[o + n_seg + n_meta:words] if n_want else None
        return d_ids, StepBatch(n_ids, d_segs, d_meta, max(s[1] + s[3] for s in segs)), d_want

    def _passes(self, entries):
        """Cut the step's entries into passes of at most ``max_rows`` rows; an entry longer than the budget continues in
        the next pass (its state carries over, exactly as between steps)."""
        cur, rows = [], 0
        for slot, tokens, want in entries:
            at = 0
            while at < len(tokens):
                take = min(len(tokens) - at, self.max_rows - rows)
                cur.append((slot, tokens[at:at + take], [w - at for w in want if at <= w < at + take]))
                rows += take
                at += take
                if rows == self.max_rows:
                    yield cur
                    cur, rows = [], 0
        if cur:
            yield cur

    # ---- decode passes as CUDA graphs
    def _graph_key(self, group, segs, want):
        """The shape of a pass that may run as a graph (None: run it eagerly): every portion is one token, logits are wanted
        for all rows or for none, and the key carries what the launches depend on besides the static buffers' contents."""
        n = len(group)
        if not self.graphs or any(len(toks) != 1 for _, toks, _ in group) or len(want) not in (0, n):
            return None
        return (n, len(want), self.model.graph_class(max(s[1] + s[3] for s in segs)))

    def _run_graphed(self, key, ids, segs, meta, want):
        g = self._step_graphs.get(key)
        if g is None:
            # first time: run eagerly (this also warms every workspace the pass allocates outside the graph's pool)
            self._step_graphs[key] = _StepGraph(2 * len(ids) + 4 * len(segs) + 2 * len(meta) + len(want), self.device)
            d_ids, batch, d_want = self._upload(ids, segs, meta, want)
            return self.model.forward_rows(d_ids, batch, d_want, self.slots)
        d_ids, batch, d_want = self._upload(ids, segs, meta, want, static=g.inputs)
        if g.graph is None:
            graph = torch.cuda.CUDAGraph()
            with graphs.capture(graph):
                g.logits = self.model.forward_rows(d_ids, batch, d_want, self.slots)
            g.graph = graph
        g.graph.replay()
        return g.logits.clone() if g.logits is not None else None

    def step(self, entries, end=(), trace=None):
        """entries: dicts ``{"id", "tokens", "want"}``; returns fp32 logits [wanted places, vocab] in the order of the entries
        and of their ``want`` lists (None if nothing is wanted)."""
        vocab = self.model.config.vocab
        todo, restore = [], []
        for e in entries:
            toks = [int(t) for t in e["tokens"]]
            if not toks:
                continue
            if min(toks) < 0 or max(toks) >= vocab:
                raise ValueError(f"request {e['id']!r}: token id outside [0, {vocab})")
            given = [int(w) for w in e.get("want", ())]
            if given and (min(given) < 0 or max(given) >= len(toks)):
                raise ValueError(f"request {e['id']!r}: wanted place outside its {len(toks)} tokens")
            # the passes produce an entry's rows in ascending order of place; `restore` puts them back into the order asked for
            order = sorted(range(len(given)), key=given.__getitem__)
            want = [given[i] for i in order]
            at = len(restore)
            restore += [0] * len(given)
            for r, g in enumerate(order):
                restore[at + g] = at + r
            slot = self.slots.slot_of(e["id"])
            if slot is None:
                slot = self.slots.alloc(e["id"])
            todo.append((slot, toks, want))
        outs = []
        for group in self._passes(todo):
            ids, segs, meta, want, row = [], [], [], [], 0
            for slot, toks, w in group:
                p0 = self.slots.reserve(slot, len(toks))
                segs.append((slot, p0, row, len(toks)))
                meta += [(slot, p0 + i) for i in range(len(toks))]
                want += [row + i for i in w]
                ids += toks
                row += len(toks)
            key = self._graph_key(group, segs, want) if trace is None else None
            if key is not None:
                logits = self._run_graphed(key, ids, segs, meta, want)
            else:
                d_ids, batch, d_want = self._upload(ids, segs, meta, want)
                logits = self.model.forward_rows(d_ids, batch, d_want, self.slots, trace=trace)
            if logits is not None:
                outs.append(logits)
        for rid in end:
            if self.slots.slot_of(rid) is not None:
                self.slots.free(rid)
        if not outs:
            return None
        logits = outs[0] if len(outs) == 1 else torch.cat(outs, 0)
        if restore != list(range(len(restore))):
            logits = logits[torch.tensor(restore, dtype=torch.int64, device=logits.device)]
        return logits

    def generate(self, prompts, max_new_tokens, chunk=None, suppress_id=-1):
        """Greedy decoding of ``prompts`` (lists of ids, any lengths) as one batch: prompts in portions of ``chunk`` tokens
        (None: whole), then one token per request per step.  Returns prompt + new tokens per request."""
        ids = list(range(len(prompts)))
        done = [0] * len(prompts)
        out = [list(p) for p in prompts]
        longest = max(len(p) for p in prompts)
        portion = chunk or longest
        nxt = [None] * len(prompts)
        while any(d < len(p) for d, p in zip(done, prompts)):
            entries = []
            for i, p in enumerate(prompts):
                if done[i] < len(p):
                    t = p[done[i]:done[i] + portion]
                    last = done[i] + len(t) == len(p)
                    entries.append({"id": i, "tokens": t, "want": [len(t) - 1] if last else []})
                    done[i] += len(t)
            logits = self.step(entries)
            if logits is not None:
                picks = ops.argmax_f32(logits, suppress_id).tolist()
                for e, tok in zip([e for e in entries if e["want"]], picks):
                    nxt[e["id"]] = tok
        for i in ids:
            out[i].append(nxt[i])
        for _ in range(max_new_tokens - 1):
            logits = self.step([{"id": i, "tokens": [out[i][-1]], "want": [0]} for i in ids])
            for i, tok in zip(ids, ops.argmax_f32(logits, suppress_id).tolist()):
                out[i].append(tok)
        for i in ids:
            self.slots.free(i)
        return out
