"""A whole decode step of a Hugging Face causal LM over a PackedStreamingCache as ONE CUDA graph.

bmx's own measurements name the per-layer Python of its packed cache (page views, partial buffers, kernel dispatch) as
what dominates a decode step end to end, not the kernel (bmx: docs/2026-07-05-authoritative-vm-results.md:193-216,
scripts/profile_decode_ab.py:316-439).  Here a single-token forward has nothing that depends on the step: the token's
position, the window lengths and the page counts live in device memory, so the model's forward -- every layer's
projections, the window append, the fused decode attention, the MLP, the head -- is captured once and replayed per token.
Steps on which the flush schedule commits a page (one in `page`) are a second graph (the slots of the new pages are
looked up on the device, the pages are quantized out of the windows, one kernel shifts the windows); the first commit of
a k2b sequence (it freezes the key basis), commits that make a pool grow and spectral packs that mix heads run through the
ordinary eager path, after which the graphs are still valid (same pools) or are captured again.
"""

from __future__ import annotations

import torch


class GraphedDecoder:
    """decoder = GraphedDecoder(model, cache); logits = decoder.step(next_ids) per token, after the prompt has been run
    through `model(prompt, past_key_values=cache)` with `cache.attach(model)` in force."""

    def __init__(self, model, cache):
        self.model, self.cache = model, cache
        self.graph: torch.cuda.CUDAGraph | None = None
        self.flush_graph: torch.cuda.CUDAGraph | None = None
        self._flush_key = None
        self.flush_replays = 0
        self._key = None
        self.ids = self.pos = self.mask = self.logits = None
        self.replays = self.eager_steps = self.captures = 0

    def _layers(self):
        return list(self.cache.layers)

    def _state_key(self):
        parts = []
        for l in self._layers():
            st = l._state
            pools = (st.pool.pages.data_ptr(),) if hasattr(st, "pool") else (st.kpool.data_ptr(), st.vpool.data_ptr())
            parts.append((pools, st.max_pages if st.committed else 0, 0 if st.rope_cos is None else st.rope_cos.data_ptr()))
        return tuple(parts)

    def _forward(self):
        # a prepared 4-D mask is passed through by the model as it is; the decode attention of one query row needs none
        return self.model(input_ids=self.ids, attention_mask=self.mask, position_ids=self.pos, past_key_values=self.cache,
                          use_cache=True).logits[:, -1]

    def _eager(self, input_ids: torch.Tensor) -> torch.Tensor:
        self.eager_steps += 1
        with torch.no_grad():
            return self.model(input_ids, past_key_values=self.cache, use_cache=True).logits[:, -1]

    def step(self, input_ids: torch.Tensor) -> torch.Tensor:
        """input_ids: (batch, 1).  Returns the logits of the new position, (batch, vocab); valid until the next step."""
        layers = self._layers()
        assert layers and layers[0]._state is not None, "run the prompt through the model first"
        S = layers[0].get_seq_length()
        if any(l.next_step_flushes() for l in layers):
            plans = [l.graph_flush_plan() for l in layers]
            rope_ok = all(l._state.rope_cos is None or S + 2 <= l._state.rope_cos.shape[0] for l in layers)
            if self.ids is None or not rope_ok or any(p is None for p in plans) or len(set(plans)) != 1:
                return self._eager(input_ids)  # the first commit (basis fit), a growing pool, another codec: the ordinary path
            key = (self._state_key(), plans[0])
            if self.flush_graph is None or self._flush_key != key:
                self._capture(flush=plans[0])
                self._flush_key = key
            self.ids.copy_(input_ids)
            self.pos.fill_(S)
            self.flush_graph.replay()
            for l in layers:
                l.advance_after_graph_flush(plans[0])
            self.flush_replays += 1
            return self.flush_logits
        need_rope = any(l._state.rope_cos is not None and S + 2 > l._state.rope_cos.shape[0] for l in layers)
        if need_rope or self.ids is None:
            # an ordinary step first: lazy one-time initialisation and a growing RoPE table stay outside any capture
            out = self._eager(input_ids)
            if self.ids is None:
                B, dev = input_ids.shape[0], input_ids.device
                self.ids = torch.zeros(B, 1, dtype=torch.long, device=dev)
                self.pos = torch.zeros(B, 1, dtype=torch.long, device=dev)
                self.mask = torch.ones(B, 1, 1, 1, dtype=torch.bool, device=dev)
            return out
        if self.graph is None or self._key != self._state_key():
            self._capture()
        self.ids.copy_(input_ids)
        self.pos.fill_(S)
        self.graph.replay()
        for l in layers:
            l.advance_after_graph_step()
        self.replays += 1
        return self.logits

    def _capture(self, flush=None) -> None:
        """Captures one single-token forward (flush: the commit every layer makes on that step, for the second graph).
        Capturing executes nothing: the step counters are not advanced."""
        layers = self._layers()
        torch.cuda.current_stream().synchronize()
        for l in layers:
            l._graph_mode, l._graph_flush = True, flush
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.no_grad(), torch.cuda.graph(graph):
                logits = self._forward()
        finally:
            for l in layers:
                l._graph_mode, l._graph_flush = False, None
        if flush is None:
            self.graph, self.logits, self._key = graph, logits, self._state_key()
        else:
            self.flush_graph, self.flush_logits = graph, logits
        self.captures += 1
