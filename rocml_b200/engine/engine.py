"""The engine: a model, its cache, and ONE step function.

``step(entries)`` runs exactly the tokens it is given, as one batch, from the cache that
earlier steps left, and returns the logits at the wanted places.  The sequences of a step
may have any lengths (whole prompts of unequal length, pieces of prompts, or one token
each); a step larger than the work space is cut into pieces internally, which changes no
result.  Steps of one token per sequence are replayed from CUDA graphs captured per batch
size and context bucket, with the batch padded up to the bucket; padding changes no result
because padded tokens carry slot -1 and every kernel skips them.

The reference has three entry points for this (one token: rocml/src/forward/mod.rs:246-387;
a chunk of one prompt: chunk_forward.rs:62-189; the chunk loop: :33-53) and no batch.
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache import SequenceCache
from ..config import load_model_spec
from ..errors import CacheError, ConfigError, KernelError, RocmlError
from ..parts import BuildEnv
from ..profile import profiler as _profiler
from .batch import BatchBuffers, HostBatch, StepBatch, pack_entries
from .model import Model

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


def _bucket(n: int, floor: int = 1) -> int:
    b = floor
    while b < n:
        b *= 2
    return b


def _ctx_bucket(n: int) -> int:
    """Context length a captured decode graph is sized for: the next multiple of 256 (of 1024 beyond
    4096).  Fine steps matter: decode attention deals its blocks out over the bucket, and blocks
    that lie past the sequences' real end do nothing."""
    step = 256 if n <= 4096 else 1024
    return max(step, -(-n // step) * step)


class Engine:
    def __init__(self, model: Model, max_tokens: int, max_slots: Optional[int] = None,
                 max_step_tokens: int = 4096, use_graphs: bool = True, max_seq_len: Optional[int] = None,
                 max_graphs: int = 8):
        """``max_graphs``: how many captured decode graphs are kept (one per batch bucket and context
        bucket, least recently used dropped first); each holds its own activations and logits."""
        self.model = model
        self.env = model.env
        self.device = model.env.device
        self.max_step_tokens = int(max_step_tokens)
        if self.max_step_tokens < 1:
            raise ConfigError("max_step_tokens must be at least 1")
        self.max_graphs = max(1, int(max_graphs))
        max_tokens = int(max_tokens)
        if max_slots is None:
            # every live sequence holds a page at least, so the pages bound the sequences (a slot costs a row
            # of the block table and, where a layer keeps fixed-size state, its state)
            max_slots = max(1, min((max_tokens + 63) // 64, 4096))
        self.use_graphs = bool(use_graphs) and model.graph_safe and self.device.type == "cuda"
        self._check_budget(max_tokens, max_slots)
        self.cache = SequenceCache(
            model.cache_requirements(), model.reads_cache_of(), max_tokens, max_slots,
            min(model.spec.max_position, max_seq_len or model.spec.max_position), self.env.act_dtype,
            self.device, self.max_step_tokens)
        self._eager: Dict[Tuple[int, int], BatchBuffers] = {}
        self._graphs: "OrderedDict[Tuple[int, int], dict]" = OrderedDict()
        self.graphs_captured = 0
        self._pool = None
        self.launches = 0          # steps issued (sub-steps counted)
        self.last_h2d_bytes = 0
        self._sampler = None
        self._device_tokens = None
        self.graph_kernel_launches = 0  # kernels run by graph replays

    # After the weights are resident: does the cache fit what is left, with head room for a step's
    # activations?  (The reference's check: rocml/src/forward/mod.rs:145-168, 768 MiB of head room,
    # rocml/src/budget/mod.rs:37.)  What a step needs is asked of the parts, so it holds for any
    # arrangement: the widest step's buffers, one more set and its logits for every captured decode
    # graph that may be kept, and the groups of fixed-size state.
    def _check_budget(self, max_tokens: int, max_slots: int) -> None:
        if self.device.type != "cuda":
            return
        esz = 4 if self.env.act_dtype == torch.float32 else 2
        per_token = state = 0
        for r, src in zip(self.model.cache_requirements(), self.model.reads_cache_of()):
            if src is not None or r is None:
                continue
            if hasattr(r, "n_kv_heads"):
                per_token += 2 * r.n_kv_heads * r.head_dim * esz
            elif hasattr(r, "shape"):
                n = 1
                for d in r.shape:
                    n *= int(d)
                state += n * torch.empty((), dtype=r.dtype).element_size() * max_slots
        step = self.model.workspace_bytes(self.max_step_tokens, min(self.max_step_tokens, max_slots))
        graphs = 0
        if self.use_graphs:
            graphs = self.max_graphs * self.model.workspace_bytes(_bucket(max_slots), _bucket(max_slots))
        headroom = (768 << 20) + step + graphs
        free, total = torch.cuda.mem_get_info(self.device)
        need = ((max_tokens + 63) // 64 * 64) * per_token + state
        if need + headroom > free:
            from ..errors import MemoryBudget
            fit = max(0, (free - headroom - state) // per_token // 64 * 64) if per_token else 0
            raise MemoryBudget(max_tokens, int(fit), (
                f"{need / 2**30:.1f} GiB of keys, values and state ({per_token} bytes per token) + "
                f"{headroom / 2**30:.1f} GiB head room (a step of {self.max_step_tokens} tokens: {step / 2**30:.2f}, "
                f"{self.max_graphs if self.use_graphs else 0} decode graphs: {graphs / 2**30:.2f}) against "
                f"{free / 2**30:.1f} GiB free of {total / 2**30:.1f} GiB"))

    # ---- construction ----------------------------------------------------------------------------
    @staticmethod
    def from_folder(folder: str, dtype: str = "bfloat16", device="cuda:0", **kw) -> "Engine":
        if dtype not in _DTYPES:
            raise ConfigError(f"dtype must be one of {sorted(set(_DTYPES))}, found {dtype!r}")
        dev = torch.device(device)
        if dev.type != "cuda":
            raise KernelError("the engine runs on a CUDA device only; there is no CPU path")
        spec = load_model_spec(folder)
        model = Model(spec, BuildEnv(dev, _DTYPES[dtype]))
        with torch.cuda.device(dev):
            model.load_folder(folder)
            return Engine(model, **kw)

    # ---- slots ---------------------------------------------------------------------------------------
    def new_sequence(self) -> int:
        return self.cache.alloc_slot()

    def release(self, slot: int) -> None:
        self.cache.free_slot(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ---- the step --------------------------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run the entries' tokens; return float32 logits [wanted places, vocab] in the order of
        the entries and of each entry's ``want`` (None when nothing is wanted).  The tensor may
        be reused by the next step: read it before stepping again.

        ``device_tokens`` (int32 on the device, one per entry) replaces the entries' token ids
        for a step of one token per sequence: the ids a sampling kernel has just written are
        fed back without passing through the host."""
        self._device_tokens = device_tokens
        if device_tokens is not None and any(len(e.tokens) != 1 for e in entries if isinstance(e, StepEntry)):
            raise RocmlError("device_tokens needs exactly one token per entry")
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        if not entries:
            return None
        seen = set()
        vocab = self.model.vocab
        for e in entries:
            if e.slot in seen:
                raise CacheError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if len(e.tokens) == 0:
                raise RocmlError(f"slot {e.slot}: a step entry needs at least one token")
            if len(e.tokens) > 64:
                arr = np.asarray(e.tokens)
                bad = arr[(arr < 0) | (arr >= vocab)][:1].tolist()
            else:
                bad = [t for t in e.tokens if not 0 <= int(t) < vocab]
            if bad:
                raise RocmlError(f"slot {e.slot}: token id {bad[0]} is outside the vocabulary of {vocab}")
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise RocmlError(f"slot {e.slot}: wanted place {w} is outside the {len(e.tokens)} tokens given")
        total = sum(len(e.tokens) for e in entries)
        if total <= self.max_step_tokens:
            pieces = [[(i, 0, len(e.tokens)) for i, e in enumerate(entries)]]
        else:
            pieces = self._cut(entries)
        # Room for everything, before anything launches.  Pages are then taken piece by piece: a
        # layer that keeps a window of keys gives pages back between the pieces of a long prompt, and
        # its group holds only a window and a piece for each sequence.
        self.cache.plan([[(entries[i].slot, b - a) for i, a, b in piece] for piece in pieces])

        with torch.cuda.device(self.device):
            outs, order = [], []
            for piece in pieces:
                slots, olds, toks, wants = [], [], [], []
                for i, a, b in piece:
                    e = entries[i]
                    slots.append(e.slot)
                    olds.append(self.cache.grow(e.slot, b - a))
                    toks.append(e.tokens[a:b])
                    w_here = sorted(w for w in set(e.want) if a <= w < b)
                    wants.append([w - a for w in w_here])
                    order.extend((i, w) for w in w_here)
                logits = self._run(slots, olds, toks, wants)
                for (i, a, b) in piece:
                    self.cache.commit(entries[i].slot, b - a)
                if logits is not None:
                    outs.append(logits)
            if not outs:
                return None
            result = outs[0] if len(outs) == 1 else torch.cat(outs, dim=0)
            wanted = [(i, w) for i, e in enumerate(entries) for w in e.want]
            if wanted != order:
                where = {key: r for r, key in enumerate(order)}
                idx = torch.tensor([where[k] for k in wanted], dtype=torch.long, device=self.device)
                result = result.index_select(0, idx)
            return result

    def _cut(self, entries):
        """Cut a step that is larger than the work space into pieces of at most
        max_step_tokens tokens, sequence after sequence, a sequence continuing in the next
        piece where it was cut (what the reference's chunk loop does for one prompt,
        rocml/src/forward/chunk_forward.rs:41-51)."""
        pieces, cur, room = [], [], self.max_step_tokens
        for i, e in enumerate(entries):
            a, n = 0, len(e.tokens)
            while a < n:
                take = min(room, n - a)
                cur.append((i, a, a + take))
                a += take
                room -= take
                if room == 0:
                    pieces.append(cur)
                    cur, room = [], self.max_step_tokens
        if cur:
            pieces.append(cur)
        return pieces

    # ---- one piece: eager launches or a graph replay ------------------------------------------------------
    def _run(self, slots, old_lens, token_lists, wants) -> Optional[torch.Tensor]:
        packed = pack_entries(slots, old_lens, token_lists, wants)
        token_ids, positions, slot_of_token, cu_q, kv_len, want_rows = packed
        T, B, W = len(token_ids), len(slots), len(want_rows)
        q_lens = [len(t) for t in token_lists]
        is_decode = all(n == 1 for n in q_lens)
        host = HostBatch(list(slots), q_lens, list(kv_len), list(want_rows))
        self.cache.flush()
        self.launches += 1
        prof = _profiler.ACTIVE
        if prof is not None:
            # a profiled step runs its kernels one by one, without a graph (rocml_b200.profile.profiler)
            with prof.step("decode" if is_decode else "prefill", q_lens, kv_len):
                return self._run_eager(packed, host, slots, q_lens, T, B, W, is_decode)
        if is_decode and self.use_graphs:
            return self._run_graph(packed, host, T, B, W)
        return self._run_eager(packed, host, slots, q_lens, T, B, W, is_decode)

    def _run_eager(self, packed, host, slots, q_lens, T, B, W, is_decode) -> Optional[torch.Tensor]:
        kv_len = packed[4]
        key = (_bucket(T, 64), _bucket(B, 8))
        if key not in self._eager:
            self._eager[key] = BatchBuffers(key[0], key[1], key[0], self.device)
        buf = self._eager[key]
        buf.fill(*packed, slots, pad_tokens=T, pad_seqs=B, pad_want=W)
        if self._device_tokens is not None:
            buf.token_ids[:B].copy_(self._device_tokens[:B], non_blocking=True)
        self.last_h2d_bytes = buf.h2d_bytes
        batch = self._batch(buf, T, B, W, max(q_lens), max(kv_len), is_decode, host)
        return self.model.forward(batch, self.cache)

    @staticmethod
    def _batch(buf: BatchBuffers, T, B, W, max_q, max_kv, is_decode, host, capturing=False) -> StepBatch:
        return StepBatch(
            n_tokens=T, n_seqs=B, n_want=W, max_q_len=max_q, max_kv_len=max_kv, is_decode=is_decode,
            token_ids=buf.token_ids, positions=buf.positions, slot_of_token=buf.slot_of_token,
            seq_slot=buf.seq_slot, cu_q=buf.cu_q, kv_len=buf.kv_len, want_rows=buf.want_rows, host=host,
            capturing=capturing)

    def _run_graph(self, packed, host, T, B, W) -> Optional[torch.Tensor]:
        kv_len = packed[4]
        b_pad = _bucket(B)
        ctx_pad = _ctx_bucket(max(kv_len))
        key = (b_pad, ctx_pad)
        g = self._graphs.get(key)
        if g is None:
            while len(self._graphs) >= self.max_graphs:
                # the least recently used bucket goes; its memory returns to the graphs' pool.  Work that
                # is still queued may read it: wait before it is released.
                _, old = self._graphs.popitem(last=False)
                torch.cuda.current_stream().synchronize()
                if old["graph"] is not None:
                    old["graph"].reset()
                old.clear()
            g = {"buffers": BatchBuffers(b_pad, b_pad, b_pad, self.device), "graph": None, "logits": None}
            self._graphs[key] = g
        else:
            self._graphs.move_to_end(key)
        buf: BatchBuffers = g["buffers"]
        buf.fill(*packed, host.seq_slots, pad_tokens=b_pad, pad_seqs=b_pad, pad_want=b_pad)
        if self._device_tokens is not None:
            buf.token_ids[:B].copy_(self._device_tokens[:B], non_blocking=True)
        self.last_h2d_bytes = buf.h2d_bytes
        if g["graph"] is None:
            # First use of this bucket: run it plainly (this also loads every kernel), then
            # capture the same launches for the next time.  Capturing executes nothing.
            batch = self._batch(buf, b_pad, b_pad, b_pad, 1, ctx_pad, True, host)
            out = self.model.forward(batch, self.cache)
            torch.cuda.current_stream().synchronize()
            graph = torch.cuda.CUDAGraph()
            cap = self._batch(buf, b_pad, b_pad, b_pad, 1, ctx_pad, True, None, capturing=True)
            from .. import kernels
            before = kernels.launch_count
            with torch.cuda.graph(graph, pool=self._pool):
                g["logits"] = self.model.forward(cap, self.cache)
            g["kernels"] = kernels.launch_count - before
            kernels.launch_count = before  # captured, not launched
            if self._pool is None:
                self._pool = graph.pool()
            g["graph"] = graph
            self.graphs_captured += 1
            return out[:W] if W else None
        g["graph"].replay()
        self.graph_kernel_launches += g["kernels"]
        return g["logits"][:W] if W else None

    # ---- generation: the engine as the loop's executor ------------------------------------------------------
    @property
    def max_seq_len(self) -> int:
        return self.cache.max_seq_len

    def capacity_tokens(self) -> int:
        return self.cache.n_pages * 64

    def capacity_slots(self) -> int:
        return self.cache.max_slots

    def launch(self, slots, tokens, params, rngs, histories, feed_from=None):
        """Enqueue a step of the sequences with their next tokens and the sampling of one token
        each, and return a handle at once.  With ``feed_from`` (the handle of the step before,
        over the same sequences in the same order) the next tokens are the ones that step
        sampled, taken on the device: ``tokens`` is not read."""
        device_tokens = None
        if feed_from is not None:
            if feed_from.n != len(slots):
                raise RocmlError("feed_from must hold one token for each sequence of the step")
            tokens = [[0]] * len(slots)
            device_tokens = feed_from.device_tokens
        if self._sampler is None:
            from ..sampling import Sampler
            self._sampler = Sampler(self.device, max_batch=max(self.cache.max_slots, 1))
        from .. import kernels
        prof = _profiler.ACTIVE
        if prof is not None:
            # the sampling belongs to the step it follows (one piece assumed; a cut prompt opens steps of its own)
            phase = "decode" if all(len(t) == 1 for t in tokens) else "prefill"
            single = sum(len(t) for t in tokens) <= self.max_step_tokens
            if single:
                with prof.step(phase, [], []):
                    logits = self.step([StepEntry(s, t, [len(t) - 1]) for s, t in zip(slots, tokens)],
                                       device_tokens=device_tokens)
                    with prof.scope(op="sampling"):
                        return self._sampler.launch(logits, params, rngs, histories,
                                                    status=kernels.status_word(self.device))
        logits = self.step([StepEntry(s, t, [len(t) - 1]) for s, t in zip(slots, tokens)], device_tokens=device_tokens)
        return self._sampler.launch(logits, params, rngs, histories, status=kernels.status_word(self.device))

    def collect(self, handle) -> List[int]:
        """Wait for a launched step and bring its token ids (nothing else) back to the host."""
        return self._sampler.collect(handle)

    def run(self, slots, tokens, params, rngs, histories) -> List[int]:
        """Step the sequences with their next tokens, sample one token each on the GPU, and
        bring the token ids back to the host."""
        return self.collect(self.launch(slots, tokens, params, rngs, histories))

    def generate(self, prompts, max_new_tokens: int = 64, sampling=None, stop_tokens=None,
                 ignore_eos: bool = False, max_batch: int = 64, on_token=None, stats=None, run_ahead: bool = True):
        """Generate for a list of prompts (token id lists).  Returns a list of Completion.
        ``sampling`` is one SamplingParams for all or a list; stop tokens default to the model's."""
        from ..sampling import SamplingParams
        from .generate import Request, generate
        if sampling is None:
            sampling = SamplingParams()
        per = sampling if isinstance(sampling, (list, tuple)) else [sampling] * len(prompts)
        reqs = [Request(list(p), max_new_tokens, sp, stop_tokens, ignore_eos) for p, sp in zip(prompts, per)]
        return generate(self, reqs, default_stop=self.model.spec.stop_tokens, max_batch=max_batch,
                        on_token=on_token, stats=stats, run_ahead=run_ahead)

    # ---- facts for measurement --------------------------------------------------------------------------------
    def kv_bytes_per_token(self) -> int:
        """Bytes of keys and values one token adds over all layers
        (rocml/src/budget/mod.rs:47-59: 2 * layers * kv heads * head size * element size)."""
        n = 0
        for g in self.cache.kv_groups:
            n += 2 * g.n_entries * g.req.n_kv_heads * g.req.head_dim * g.k.element_size()
        return n
