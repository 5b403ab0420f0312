"""Rollout engine: continuous batching over a paged KV cache, running the SAME ``DecoderLM``
the trainer runs (the reference needs vLLM + a Megatron-in-vLLM wrapper for this,
ISO/runtimes/vllm/gptmodel_vllm.py:642-721; here the engine is ~400 lines around the shared model).

A step is one forward over a flat token batch: the decode tokens of running sequences first,
then (chunked) prefill tokens of admitted sequences, up to ``max_num_batched_tokens``. Every
token goes through the same kernels whatever the mix, which is what makes a token's logprob
independent of the batch it was computed in.
"""

from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field

import torch

from ..models.decoder import DecoderLM, ForwardCtx
from ..ops import functional as F
from ..ops.functional import PAGE
from .kv_cache import KVCache
from .sampler import Sampler, SamplingParams
from .sampler import needs_history as _needs_history


@dataclass
class EngineConfig:
    max_num_seqs: int = 1024
    max_num_batched_tokens: int = 8192
    num_kv_pages: int = 0                # 0 = size from gpu_memory_utilization
    gpu_memory_utilization: float = 0.8
    max_model_len: int = 0               # 0 = model max_position
    eos_token_id: int | None = None
    seed: int = 0
    enable_prefix_caching: bool = False  # full KV pages are kept after their request and reused by later requests with the
                                         # same leading tokens (engine/prefix_cache.py); dropped at every weight sync
    prefix_cache_state_mb: int = 1024    # models with recurrent layers: budget of the boundary states kept beside the pages
    use_cuda_graph: bool = True
    share_prompt_pages: bool = True      # samples of one prompt share its full KV pages (not a cache: freed with the requests)
    share_recurrent_state: bool = False  # models with GatedDeltaNet layers: siblings also start from the leader's recurrent
                                         # state at the shared boundary (a snapshot taken when its prefill gets there)


@dataclass
class Sequence:
    seq_id: int
    prompt_ids: list[int]
    params: SamplingParams
    output_ids: list[int] = field(default_factory=list)
    logprobs: list[float] = field(default_factory=list)
    pages: list[int] = field(default_factory=list)
    num_computed: int = 0          # tokens whose K/V are in the cache
    finished: bool = False
    stop_reason: str | None = None
    request_index: int = 0
    arrival: float = 0.0
    # Samples of one prompt: a sequence whose prompt equals an earlier one's of the same generate() call takes the
    # leader's full prompt pages (all but the page holding the last prompt token) instead of recomputing them.
    leader: "Sequence | None" = None
    shared_tokens: int = 0
    snapshot_at: int = 0           # leader of a model with recurrent layers: its prefill stops here once, for a state snapshot
    snapshot_users: int = 0
    # vision-language requests: prompt positions of the image placeholder tokens, the vision tower's row for each of them
    # (on the engine's device), and a digest of the pixels (two requests share pages only if their images are the same)
    mm_pos: list[int] | None = None
    mm_feats: torch.Tensor | None = None
    mm_key: bytes | None = None
    prompt_logprobs: list | None = None     # requested with SamplingParams.prompt_logprobs: [None, lp(token 1 | token 0), ...]

    @property
    def tokens(self) -> list[int]:
        return self.prompt_ids + self.output_ids

    @property
    def length(self) -> int:
        return len(self.prompt_ids) + len(self.output_ids)

    @property
    def last_token(self) -> int:
        return self.output_ids[-1] if self.output_ids else self.prompt_ids[-1]


@dataclass
class RequestOutput:
    prompt_ids: list[int]
    response_ids: list[int]
    response_logprobs: list[float]
    stop_reason: str
    prompt_logprobs: list | None = None


class Scheduler:
    """Decode-first continuous batching with chunked prefill and recompute-preemption."""

    def __init__(self, cfg: EngineConfig, cache: KVCache):
        self.cfg = cfg
        self.cache = cache
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self.preemptions = 0
        self.shared_prompt_tokens = 0       # prompt tokens taken from a leader's pages instead of being prefilled
        self.can_adopt = None               # engine hooks for models with recurrent state: (sibling, leader) -> bool / None
        self.adopt_hook = None
        self.prefix = None                  # PrefixCache when prefix caching is on
        self.prefix_hit_hook = None         # (sequence, chain key of the matched prefix): recurrent state is loaded here

    def add(self, seq: Sequence) -> None:
        self.waiting.append(seq)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _ensure_pages(self, seq: Sequence, upto: int) -> bool:
        need = (upto + PAGE - 1) // PAGE - len(seq.pages)
        if need <= 0:
            return True
        if not self.cache.allocator.can_alloc(need) and self.prefix is not None:
            self.prefix.evict(need - self.cache.allocator.num_free)      # cached pages nobody reads go before a preemption
        if not self.cache.allocator.can_alloc(need):
            return False
        seq.pages += self.cache.allocator.alloc(need)
        return True

    def _preempt(self, seq: Sequence) -> None:
        if self.prefix is not None and seq.mm_feats is None:
            self.prefix.insert(seq.tokens, seq.pages, seq.num_computed)  # the recompute may find them again
        self.cache.allocator.release(seq.pages)
        seq.pages = []
        seq.num_computed = 0
        seq.leader = None
        self.waiting.appendleft(seq)

    @staticmethod
    def _chunk(s: Sequence, budget: int) -> int:
        """Tokens of ``s`` to prefill now: what is left, within the budget, and not across a pending snapshot boundary."""
        n = min(s.length - s.num_computed, budget)
        if s.snapshot_at and s.num_computed < s.snapshot_at:
            n = min(n, s.snapshot_at - s.num_computed)
        return n

    def schedule(self):
        """Returns (decode_seqs, prefill list of (seq, start, n))."""
        budget = self.cfg.max_num_batched_tokens
        decode: list[Sequence] = []
        # running sequences that have their whole context cached decode one token
        running = [s for s in self.running if s.num_computed == s.length - 1]
        still_prefilling = [s for s in self.running if s.num_computed < s.length - 1]
        for s in running:
            while s in self.running and not self._ensure_pages(s, s.length):
                # out of pages: preempt the most recently admitted sequence (possibly s itself);
                # it is recomputed from its tokens when pages free up
                victims = [v for v in self.running if v.pages]
                if len(victims) <= 1 and victims == [s]:
                    raise RuntimeError("KV cache too small for a single sequence")
                v = victims[-1]
                self.running.remove(v)
                if v in still_prefilling:
                    still_prefilling.remove(v)
                if v in decode:
                    decode.remove(v)
                    budget += 1
                self.preemptions += 1
                self._preempt(v)
            if s in self.running:
                decode.append(s)
                budget -= 1
        prefill = []
        for s in still_prefilling:
            if budget <= 0:
                break
            n = self._chunk(s, budget)
            if not self._ensure_pages(s, s.num_computed + n):
                continue
            prefill.append((s, s.num_computed, n))
            budget -= n
        i = 0
        while i < len(self.waiting) and budget > 0 and len(self.running) < self.cfg.max_num_seqs:
            s = self.waiting[i]
            if s.leader is not None:
                ld = s.leader
                if s.pages or s.num_computed or ld.finished or len(ld.pages) * PAGE < s.shared_tokens:
                    s.leader = None                      # the leader's pages are gone (or s was preempted): on its own
                elif ld.num_computed < s.shared_tokens:
                    i += 1                               # the shared prompt pages are not written yet: later sequences first
                    continue
                elif self.can_adopt is not None and not self.can_adopt(s, ld):
                    i += 1                               # the leader's recurrent state at the boundary is not snapshotted yet
                    continue
                else:
                    s.pages = list(ld.pages[:s.shared_tokens // PAGE])
                    self.cache.allocator.share(s.pages)
                    s.num_computed = s.shared_tokens
                    s.leader = None
                    self.shared_prompt_tokens += s.shared_tokens
                    if self.adopt_hook is not None:
                        self.adopt_hook(s, ld)
            if self.prefix is not None and s.leader is None and not s.pages and s.num_computed == 0 and s.mm_feats is None \
                    and s.prompt_logprobs is None:
                pages, key = self.prefix.match(s.tokens)
                if pages:
                    s.pages, s.num_computed = pages, len(pages) * PAGE
                    if self.prefix_hit_hook is not None:
                        self.prefix_hit_hook(s, key)
            n = self._chunk(s, budget)
            if not self._ensure_pages(s, s.num_computed + n):
                break
            del self.waiting[i]
            self.running.append(s)
            prefill.append((s, s.num_computed, n))
            budget -= n
        return decode, prefill

    def finish(self, seq: Sequence) -> None:
        if self.prefix is not None and seq.mm_feats is None:      # pages are keyed by tokens alone: image prompts stay out
            self.prefix.insert(seq.tokens, seq.pages, seq.num_computed)
        self.cache.allocator.release(seq.pages)
        seq.pages = []
        self.running.remove(seq)


class LLMEngine:
    def __init__(self, model: DecoderLM, cfg: EngineConfig | None = None):
        self.model = model
        self.mcfg = model.cfg
        self.cfg = cfg or EngineConfig()
        self.device = model.device_
        self.max_len = self.cfg.max_model_len or self.mcfg.max_position
        n_pages = self.cfg.num_kv_pages or self._auto_pages()
        self.cache = KVCache(self.mcfg, n_pages, self.device, tp=model.ps.tp, layer_ids=model.layer_ids)
        self.scheduler = Scheduler(self.cfg, self.cache)
        self.sampler = Sampler(self.device, self.cfg.seed, self.mcfg.logprob_leaves)
        self._next_id = 0
        self.detokenize = None          # ids -> text, set by whoever owns a tokenizer; needed only for stop STRINGS
        self.paused = False
        self.asleep = False
        self.stats = {"steps": 0, "tokens": 0, "prefill_tokens": 0, "decode_tokens": 0, "preemptions": 0,
                      "h2d_bytes": 0, "d2h_bytes": 0}
        self._graphs: dict = {}
        self._ep_lockstep = model.ps.ep > 1 and self.mcfg.has_moe
        self._global_work = False
        self._inflight: dict | None = None        # a decode step launched but not yet read back
        self._res_host: list = [None, None]       # pinned result buffers, alternating
        self._res_parity = 0
        if self.device.type == "cuda":
            from ..ops import _native

            _native.lib().ix_init()   # status word allocated before any stream capture
        self.gdn_state = None
        if self.mcfg.has_gdn:
            from .gdn_state import GDNStatePool

            self.gdn_state = GDNStatePool(self.mcfg, self.cfg.max_num_seqs, self.device, tp=model.ps.tp)
            if self.cfg.share_prompt_pages and self.cfg.share_recurrent_state:
                self.scheduler.can_adopt = lambda s, ld: self.gdn_state.has_snapshot(ld.seq_id)
                self.scheduler.adopt_hook = lambda s, ld: self.gdn_state.adopt(s.seq_id, ld.seq_id)
        self.prefix_cache = None
        if self.cfg.enable_prefix_caching:
            from .prefix_cache import BoundaryStates, PrefixCache

            boundary = BoundaryStates(self.cfg.prefix_cache_state_mb << 20) if self.gdn_state is not None else None
            self.prefix_cache = self.scheduler.prefix = PrefixCache(self.cache.allocator, boundary)
            if boundary is not None:
                self.scheduler.prefix_hit_hook = self._resume_from_boundary

    def _auto_pages(self) -> int:
        per_page = KVCache.bytes_per_page(self.mcfg, self.model.ps.tp)
        if per_page == 0:
            return 1
        if self.device.type == "cuda":
            free, _total = torch.cuda.mem_get_info(self.device)
            budget = int(free * self.cfg.gpu_memory_utilization)
        else:
            budget = 256 << 20
        want = self.cfg.max_num_seqs * ((self.max_len + PAGE - 1) // PAGE)
        return max(2, min(want, budget // per_page))

    def _h2d(self, t: torch.Tensor) -> torch.Tensor:
        """Stage a host tensor in pinned memory and copy it to the engine's device (counted)."""
        self.stats["h2d_bytes"] += t.numel() * t.element_size()
        if self.device.type != "cuda":
            return t
        return t.pin_memory().to(self.device, non_blocking=True)

    # ------------------------------------------------------------------ lifecycle
    def sleep(self, tags: list[str] | None = None) -> None:
        """Release the KV pools (and recurrent state). Weights stay resident."""
        self._drain_inflight()
        assert not self.scheduler.has_work(), "sleep with requests in flight"
        self._drop_prefix_cache()
        self._graphs.clear()      # graphs hold the pool addresses; they are re-captured after wake-up
        self.cache.sleep()
        if self.prefix_cache is not None:
            self.prefix_cache.alloc = self.cache.allocator       # sleep starts a fresh allocator
        if self.gdn_state is not None:
            self.gdn_state.invalidate("sleep_wake")
        self.asleep = True

    def wake_up(self, tags: list[str] | None = None) -> None:
        self.cache.wake()
        self.asleep = False

    def reset_prefix_cache(self) -> None:
        """Called at every weight sync. Cached prefixes (pages and boundary states) are dropped, after which the KV cache
        checks that no page holds old-weight state; recurrent state is dropped."""
        self._drain_inflight()
        self._drop_prefix_cache()
        self.cache.invalidate("weight_sync")
        if self.gdn_state is not None:
            self.gdn_state.invalidate("weight_sync")

    def _drop_prefix_cache(self) -> None:
        if self.prefix_cache is not None:
            self.prefix_cache.clear()
            self.stats["prefix_cache_drops"] = self.stats.get("prefix_cache_drops", 0) + 1

    def _resume_from_boundary(self, s: Sequence, key: bytes) -> None:
        """A sequence of a model with recurrent layers matched a cached prefix: its state row starts from the boundary
        state stored for that prefix. A leader whose siblings wait for a snapshot at this very boundary gives it now
        (its prefill will not pass the boundary again)."""
        self.gdn_state.load_row(s.seq_id, self.prefix_cache.boundary.get(key))
        if s.snapshot_at and s.num_computed == s.snapshot_at and s.snapshot_users > 0:
            self.gdn_state.snapshot(s.seq_id, s.snapshot_users)

    def _note_progress(self, s: Sequence, prefill: bool) -> None:
        """After a step that advanced ``s``: list its newly full pages (a later request may match them while this one
        still runs), and for a model with recurrent layers keep the state at a page boundary the sequence stands on
        exactly (its open chunk is empty there)."""
        pc = self.prefix_cache
        if pc is None or s.num_computed < PAGE or not (prefill or s.num_computed % PAGE == 0) or s.mm_feats is not None:
            return
        if pc.boundary is not None:
            if s.num_computed % PAGE or s.seq_id not in self.gdn_state.row_of:
                return
            from .prefix_cache import chain_keys

            key = chain_keys(s.tokens, s.num_computed // PAGE)[-1]
            if key not in pc.boundary:
                pc.boundary.put(key, self.gdn_state.clone_row(s.seq_id))
        pc.insert(s.tokens, s.pages, s.num_computed)

    def invalidation_counts(self) -> dict:
        """{state id of the contract: {event: times the state was really invalidated}}."""
        out = {"engine_kv_cache": dict(self.cache.invalidations)}
        if self.gdn_state is not None:
            out["gdn_recurrent_state"] = dict(self.gdn_state.invalidations)
        return out

    def pause_generation(self) -> None:
        self.paused = True

    def resume_generation(self) -> None:
        self.paused = False

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt_ids: list[int], params: SamplingParams, request_index: int = 0, mm: dict | None = None) -> Sequence:
        """``mm``: ``{"pixel_values": [patches, dim], "image_grid_thw": [images, 3], "positions": optional list}`` for a
        prompt with image placeholder tokens (``positions``: where they are; default: every token equal to the model's
        ``image_token_id``). The vision tower runs here, once per request."""
        if len(prompt_ids) == 0:
            raise ValueError("empty prompt")
        if len(prompt_ids) >= self.max_len:
            raise ValueError(f"prompt of {len(prompt_ids)} tokens exceeds max_model_len={self.max_len}")
        seq = Sequence(self._next_id, list(prompt_ids), params, request_index=request_index, arrival=time.time())
        self._next_id += 1
        if mm is not None and mm.get("pixel_values") is not None and mm["pixel_values"].shape[0]:
            self._attach_images(seq, mm)
        if params.prompt_logprobs is not None:
            seq.prompt_logprobs = [None] * len(prompt_ids)
        if self.prefix_cache is not None and self.prefix_cache.boundary is not None:
            # recurrent layers: the prefill stops once at the last full page of the prompt, so that the state there can be
            # kept for later requests that share the prompt
            seq.snapshot_at = ((len(prompt_ids) - 1) // PAGE) * PAGE
        self.scheduler.add(seq)
        return seq

    @torch.no_grad()
    def _attach_images(self, seq: Sequence, mm: dict) -> None:
        import hashlib

        tower = getattr(self.model, "vision", None)
        if tower is None:
            raise ValueError(f"model {self.mcfg.name!r} has no vision tower: it cannot take image inputs")
        pv, grid = mm["pixel_values"], mm["image_grid_thw"]
        tok = self.mcfg.image_token_id
        pos = list(mm["positions"]) if mm.get("positions") is not None else [i for i, t in enumerate(seq.prompt_ids) if t == tok]
        feats = tower.encode(pv, grid)
        if feats.shape[0] != len(pos):
            raise ValueError(f"the prompt has {len(pos)} image placeholder tokens, the images give {feats.shape[0]} feature rows")
        if any(seq.prompt_ids[p] != tok for p in pos) or sorted(pos) != pos:
            raise ValueError("image positions must be ascending and point at image placeholder tokens")
        seq.mm_pos, seq.mm_feats = pos, feats
        seq.mm_key = hashlib.blake2b(pv.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes()
                                     + grid.detach().cpu().to(torch.int64).numpy().tobytes(), digest_size=16).digest()

    @staticmethod
    def _image_rows_of_chunk(s: Sequence, start: int, n: int, row: int):
        """Batch rows and feature rows of the image placeholder tokens of ``s`` inside its prefill chunk [start, start+n)."""
        import bisect

        k0, k1 = bisect.bisect_left(s.mm_pos, start), bisect.bisect_left(s.mm_pos, start + n)
        return [row + (p - start) for p in s.mm_pos[k0:k1]], s.mm_feats[k0:k1]

    @torch.no_grad()
    def step(self) -> list[Sequence]:
        """Run one scheduler step; returns the sequences that finished in it.

        Graph-replayed decode steps run ONE STEP AHEAD of the host: the step's sampled tokens stay on the device and
        feed the next replay directly, which is launched before the host reads them back; the host then appends the
        previous step's tokens while the GPU is already busy. A sequence that turns out to have stopped (EOS) has one
        surplus token computed, which is dropped. Results therefore come back one call later than they were launched."""
        if self._ep_lockstep:
            # every MoE layer is a collective over the EP group: ranks step together, and a rank with nothing to do
            # still serves its experts to the others
            mine = self.scheduler.has_work()
            self._global_work = self._ep_vote(mine)
            if not self._global_work:
                return []
            if not mine:
                self.model.ep_idle_forward()
                return []
        if self._inflight is not None:
            prev = self._inflight
            nxt = self._launch_ahead(prev) if self._can_run_ahead(prev) else None
            self._inflight = nxt
            return self._finalize(prev)
        decode, prefill = self.scheduler.schedule()
        if not decode and not prefill:
            return []
        if not prefill and self._graphs_enabled() and not any(_needs_history(s.params) for s in decode):
            # (a request whose sampling looks at its own tokens cannot run ahead of the host: the token in flight is part
            # of that history)
            self._inflight = self._launch_decode(decode, ahead=False)
            return []
        G = self.model.hq // self.model.hkv
        tq = PAGE // G
        ids, pos, slots, items, bt_rows, sample_rows, sample_seqs = [], [], [], [], [], [], []
        mm_rows, mm_feats = [], []
        row = 0
        for s in decode:
            p = s.length - 1
            ids.append(s.last_token)
            pos.append(p)
            slots.append(s.pages[p // PAGE] * PAGE + p % PAGE)
            items.append((row, 1, p, p + 1, len(bt_rows), 0, 0, 0))
            bt_rows.append(s.pages)
            sample_rows.append(row)
            sample_seqs.append(s)
            row += 1
        for s, start, n in prefill:
            toks = s.tokens
            ids += toks[start:start + n]
            pos += range(start, start + n)
            slots += self.cache.slots_for(s.pages, start, n)
            bt = len(bt_rows)
            bt_rows.append(s.pages)
            for t0 in range(0, n, tq):
                items.append((row + t0, min(tq, n - t0), start + t0, start + n, bt, 0, 0, 0))
            if start + n == s.length:
                sample_rows.append(row + n - 1)
                sample_seqs.append(s)
            if s.mm_feats is not None:
                r, f = self._image_rows_of_chunk(s, start, n, row)
                if r:
                    mm_rows += r
                    mm_feats.append(f)
            row += n
        maxp = max(len(b) for b in bt_rows)
        bt = torch.zeros(len(bt_rows), maxp, dtype=torch.int32)
        for i, b in enumerate(bt_rows):
            bt[i, :len(b)] = torch.tensor(b, dtype=torch.int32)
        fc = ForwardCtx(
            positions=self._h2d(torch.tensor(pos, dtype=torch.int32)),
            meta=F.AttnMeta(self._h2d(torch.tensor(items, dtype=torch.int32).reshape(-1, 8)), self._h2d(bt)),
            slots=self._h2d(torch.tensor(slots, dtype=torch.int64)),
            kv=self.cache.pools,
            site="engine_decode" if not prefill else "engine_prefill",
        )
        if self.gdn_state is not None:
            fc.gdn_meta = self.gdn_state.step_meta(decode, prefill)
            fc.kv = self.gdn_state.merge_into(self.cache.pools)
        if mm_rows:
            fc.mm = (self._h2d(torch.tensor(mm_rows, dtype=torch.int64)), torch.cat(mm_feats, 0))
        hidden = self.model(self._h2d(torch.tensor(ids, dtype=torch.int64)), fc)
        if any(s.prompt_logprobs is not None for s, _, _ in prefill):
            self._fill_prompt_logprobs(hidden, prefill, len(decode))
        for s in decode:
            s.num_computed += 1
            self._note_progress(s, False)
        for s, start, n in prefill:
            s.num_computed = start + n
            if s.snapshot_at and start + n == s.snapshot_at and self.gdn_state is not None and s.snapshot_users > 0:
                self.gdn_state.snapshot(s.seq_id, s.snapshot_users)          # the siblings of this prompt start from here
            self._note_progress(s, True)
        self.stats["steps"] += 1
        self.stats["tokens"] += row
        self.stats["decode_tokens"] += len(decode)
        self.stats["prefill_tokens"] += row - len(decode)
        if not sample_rows:
            return []
        rows = self._h2d(torch.tensor(sample_rows, dtype=torch.int64))
        logits = self.model.logits(hidden.index_select(0, rows))
        return self._sample_and_finish(logits, sample_seqs)

    def _fill_prompt_logprobs(self, hidden: torch.Tensor, prefill: list, first_row: int, chunk_rows: int = 1024) -> None:
        """Log-probability of every prompt token given the tokens before it, for the requests that asked: row t of a
        prefill chunk predicts token t + 1, so the rows whose successor is still a prompt token are scored with the
        kernel that scores sampled tokens. (A prompt cut into prefill chunks loses nothing: the row that predicts a
        chunk's first token is the last row of the chunk before it.)"""
        row = first_row
        for s, start, n in prefill:
            if s.prompt_logprobs is not None:
                P = len(s.prompt_ids)
                hi = min(start + n, P - 1)                      # rows start .. hi-1 predict prompt tokens start+1 .. hi
                for lo in range(start, hi, chunk_rows):
                    up = min(hi, lo + chunk_rows)
                    if all(v is not None for v in s.prompt_logprobs[lo + 1:up + 1]):
                        continue                                # a recomputed (preempted) sequence: already filled
                    logits = self.model.logits(hidden[row + (lo - start):row + (up - start)])
                    if self.model.ps.tp > 1:
                        from ..parallel.tp import column_parallel_gather

                        logits = column_parallel_gather(logits, self.model.ps)
                    tg = self._h2d(torch.tensor(s.prompt_ids[lo + 1:up + 1], dtype=torch.int64))
                    lp, _ = F.token_logprobs(logits, tg, self.mcfg.logprob_leaves)
                    s.prompt_logprobs[lo + 1:up + 1] = lp.tolist()
            row += n

    def _sample_and_finish(self, logits: torch.Tensor, sample_seqs: list[Sequence]) -> list[Sequence]:
        if self.model.ps.tp > 1:
            from ..parallel.tp import column_parallel_gather

            logits = column_parallel_gather(logits, self.model.ps)
        hist = [(s.prompt_ids, s.output_ids) for s in sample_seqs] if any(_needs_history(s.params) for s in sample_seqs) else None
        tokens, lps = self.sampler(logits, [s.params for s in sample_seqs], histories=hist, eos_token_id=self.cfg.eos_token_id)
        self.stats["d2h_bytes"] += tokens.numel() * 8 + lps.numel() * 4
        tokens, lps = tokens.tolist(), lps.tolist()
        finished: list[Sequence] = []
        eos = self.cfg.eos_token_id
        for s, tok, lp in zip(sample_seqs, tokens, lps):
            s.output_ids.append(tok)
            s.logprobs.append(lp)
            if (not s.params.ignore_eos and eos is not None and tok == eos) or tok in s.params.stop_token_ids \
                    or self._hit_stop_string(s):
                s.finished, s.stop_reason = True, "stop"
            elif len(s.output_ids) >= s.params.max_generate_length or s.length >= self.max_len:
                s.finished, s.stop_reason = True, "length"
            if s.finished:
                if self.gdn_state is not None:
                    self.gdn_state.release(s.seq_id)
                self.scheduler.finish(s)
                finished.append(s)
        return finished

    # ------------------------------------------------------------------ CUDA-graph decode
    def _graphs_enabled(self) -> bool:
        """Decode steps are replayed from a CUDA graph unless the model has a layer whose decode is not host-free yet
        (expert-parallel MoE, GatedDeltaNet state slots). Tensor parallelism: the row-parallel GEMMs must be
        served by the fused peer-memory kernel (its graph form reads the epoch from a device word); with the NCCL
        transport the step stays eager."""
        if not (self.cfg.use_cuda_graph and self.device.type == "cuda") or self.mcfg.has_gdn:
            return False
        ps = self.model.ps
        if self.mcfg.has_moe:
            # single-rank experts build their routing tables on the device (ops/moe.py DispatchPlan): host-free.
            # Expert parallelism exchanges counts through handshakes whose epochs are kernel arguments: eager.
            from ..ops import moe as moe_ops

            i = next((j for j in self.model.layer_ids if self.mcfg.has_moe), None)
            if ps.ep > 1 or i is None:
                return False
            gu, dn = self.model.p(f"layers.{i}.moe.experts.gate_up"), self.model.p(f"layers.{i}.moe.experts.down")
            if not moe_ops._experts_fn_ok(gu, gu, dn):
                return False
        if ps.tp > 1:
            from ..parallel import tp_fused

            return tp_fused.get(ps.tp_group) is not None and bool(getattr(self.mcfg, "tp_invariant", False))
        return True

    def _launch_decode(self, decode: list[Sequence], ahead: bool) -> dict:
        """Enqueue (copy, graph replay, sampling, device-side token feedback, D2H of the results) for one decode step
        and return without waiting. ``ahead``: a token of every sequence is still in flight, so positions are one
        further than the host's view and the input tokens are already in the graph's id buffer."""
        from .cuda_graph import DecodeGraph

        B = len(decode)
        W = (self.max_len + PAGE - 1) // PAGE
        g = self._graphs.get(B)
        if g is None:
            g = DecodeGraph(self, B, W)
            self._graphs[B] = g
        off = 1 if ahead else 0
        pos, slots, items, bt_rows = [], [], [], []
        for i, s in enumerate(decode):
            p = s.length - 1 + off
            pos.append(p)
            slots.append(s.pages[p // PAGE] * PAGE + p % PAGE)
            items.append((i, 1, p, p + 1, i, 0, 0, 0))
            bt_rows.append(s.pages)
        g.fill(None if ahead else [s.last_token for s in decode], pos, slots, items, bt_rows)
        if g.graph is None:
            g.dev.copy_(g.host)
            g.capture()
        logits = g.run()
        if self.model.ps.tp > 1:          # vocabulary shards -> full rows (bytes only; outside the graph)
            from ..parallel.tp import column_parallel_gather

            logits = column_parallel_gather(logits, self.model.ps)
        tokens, lps = self.sampler(logits, [s.params for s in decode])
        g.ids.copy_(tokens)                       # next replay's input, device to device
        k = self._res_parity = self._res_parity ^ 1
        if self._res_host[k] is None or self._res_host[k][0].numel() < B:
            self._res_host[k] = (torch.zeros(max(B, 64), dtype=torch.int64).pin_memory(), torch.zeros(max(B, 64), dtype=torch.float32).pin_memory())
        ht, hl = self._res_host[k]
        ht[:B].copy_(tokens, non_blocking=True)
        hl[:B].copy_(lps, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.stats["steps"] += 1
        self.stats["tokens"] += B
        self.stats["decode_tokens"] += B
        self.stats["d2h_bytes"] += B * 12
        return {"seqs": list(decode), "tokens": ht, "lps": hl, "event": ev, "B": B}

    def _can_run_ahead(self, prev: dict) -> bool:
        """The next step may be launched before the previous one is read back only if its batch is known now: nothing
        waits to be admitted, no sequence ends by length with the token in flight, and every sequence has a KV slot for it."""
        if self.paused or self.scheduler.waiting or not self._graphs_enabled():
            return False
        seqs = prev["seqs"]
        if len(seqs) != len(self.scheduler.running) or any(s.finished for s in seqs):
            return False
        for s in seqs:
            if len(s.output_ids) + 1 >= s.params.max_generate_length or s.length + 1 >= self.max_len:
                return False
        for s in seqs:
            if not self.scheduler._ensure_pages(s, s.length + 1):
                return False
        return True

    def _launch_ahead(self, prev: dict) -> dict:
        return self._launch_decode(prev["seqs"], ahead=True)

    def _hit_stop_string(self, s) -> bool:
        """Stop strings: decode a tail of the output long enough to contain the longest stop string and look for them.
        Needs ``self.detokenize`` (ids -> text); the matched text stays in the output, as with a stop token."""
        stops = s.params.stop
        if not stops or self.detokenize is None:
            return False
        longest = max(len(x) for x in stops)
        tail = s.output_ids[-min(len(s.output_ids), 4 * longest + 8):]        # generous: a token is at least one character
        return any(x in self.detokenize(tail) for x in stops)

    def _finalize(self, rec: dict) -> list[Sequence]:
        """Wait for a launched step's results and apply them (append token, stop checks, release)."""
        rec["event"].synchronize()
        B = rec["B"]
        tokens, lps = rec["tokens"][:B].tolist(), rec["lps"][:B].tolist()
        finished: list[Sequence] = []
        eos = self.cfg.eos_token_id
        for s, tok, lp in zip(rec["seqs"], tokens, lps):
            if s.finished:                      # stopped (or was aborted) while this surplus step was in flight
                continue
            s.num_computed += 1                 # the step cached the K/V of the token it consumed
            s.output_ids.append(tok)
            s.logprobs.append(lp)
            if (not s.params.ignore_eos and eos is not None and tok == eos) or tok in s.params.stop_token_ids \
                    or self._hit_stop_string(s):
                s.finished, s.stop_reason = True, "stop"
            elif len(s.output_ids) >= s.params.max_generate_length or s.length >= self.max_len:
                s.finished, s.stop_reason = True, "length"
            if s.finished:
                if self.gdn_state is not None:
                    self.gdn_state.release(s.seq_id)
                self.scheduler.finish(s)
                finished.append(s)
        return finished

    def _ep_vote(self, have: bool) -> bool:
        import torch.distributed as dist

        t = torch.tensor([1 if have else 0], dtype=torch.int32, device=self.device if self.device.type == "cuda" else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.model.ps.ep_group)
        return bool(int(t))

    def _drain_inflight(self) -> None:
        if self._inflight is not None:
            rec, self._inflight = self._inflight, None
            self._finalize(rec)

    def link_samples(self, seqs: list[Sequence]) -> int:
        """Among requests that were just added together, make every sequence whose prompt equals an earlier one's a
        sibling of it: the n samples of a prompt then read the first one's full prompt pages instead of prefilling them
        again (K/V rows do not depend on the batch they are computed in, so the bits are the same) and prefill only
        the page that holds the last prompt token. Returns the number of siblings made. Models with recurrent layers are
        linked only with ``share_recurrent_state``: the leader's prefill then stops once at the shared boundary, its
        recurrent state is snapshotted there, and a sibling starts from the snapshot."""
        recurrent = self.mcfg.has_gdn
        if not self.cfg.share_prompt_pages or (recurrent and not self.cfg.share_recurrent_state):
            return 0
        leaders: dict = {}
        n = 0
        for s in seqs:
            if s.num_computed or s.pages or s.output_ids:
                continue                                        # already under way
            if s.prompt_logprobs is not None:
                continue                                        # every prompt row of such a request must be computed
            ld = leaders.setdefault((tuple(s.prompt_ids), s.mm_key), s)
            shared = ((len(s.prompt_ids) - 1) // PAGE) * PAGE   # a multiple of the GatedDeltaNet chunk too: no open chunk there
            if ld is not s and shared > 0:
                s.leader, s.shared_tokens = ld, shared
                if recurrent:
                    ld.snapshot_at, ld.snapshot_users = shared, ld.snapshot_users + 1
                n += 1
        return n

    def generate(self, prompts: list[list[int]], params: SamplingParams | list[SamplingParams], mm: list | None = None) -> list[RequestOutput]:
        """Blocking batch generation; outputs are in prompt order. ``mm``: per prompt, the image inputs of ``add_request``
        or None."""
        if self.asleep:
            raise RuntimeError("engine is asleep; call wake_up() first")
        plist = params if isinstance(params, list) else [params] * len(prompts)
        mlist = mm if mm is not None else [None] * len(prompts)
        seqs = [self.add_request(p, sp, i, mm=m) for i, (p, sp, m) in enumerate(zip(prompts, plist, mlist))]
        self.link_samples(seqs)
        while True:
            if self.paused:
                time.sleep(0.001)
                continue
            if not self._ep_lockstep and not self.scheduler.has_work():
                break
            self.step()
            if self._ep_lockstep and not self._global_work:
                break
        return [RequestOutput(s.prompt_ids, s.output_ids, s.logprobs, s.stop_reason or "length", s.prompt_logprobs) for s in seqs]
