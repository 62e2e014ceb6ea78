"""What the sequence-step language models share on the host: the entry-point class (loading, step(), generate() through
serving.StepScheduler) and the replay of decode-only steps from a CUDA graph.

A decoder class provides `step(tokens, pos, slot, cache, want_rows, collect, portions, one_row_each)` and `new_cache(...)`; its model
class names it in `decoder_class`, its configuration in `config_class`, and the function that turns a checkpoint's tensors into
its weight structure in `weights_from_state_dict`.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .. import lib, seqlib


def portion_starts(decoder, T: int, slot: torch.Tensor, portions: Optional[Sequence], one_row_each: bool = False):
    """(device int32 [P + 1] with the first row of every request's portion followed by T, P): what the recurrences walk. portions:
    the host's [(first_row, n_rows, slot, first_pos)]; without it the starts are derived from the slots (a host round trip: tests,
    debugging). When every row is a request of its own the answer is a cached arange (`decoder._arange`)."""
    if not one_row_each:
        if portions is None:
            s = slot.cpu()
            starts = [0] + [i for i in range(1, T) if s[i] != s[i - 1]]
        else:
            starts = [p[0] for p in portions]
        one_row_each = len(starts) == T
    if one_row_each:
        if getattr(decoder, "_arange", None) is None or decoder._arange.numel() < T + 1:
            decoder._arange = torch.arange(max(T + 1, 65), device=decoder.device, dtype=torch.int32)
        return decoder._arange, T
    rb = torch.tensor(starts + [T], dtype=torch.int32)
    if torch.device(decoder.device).type == "cuda":
        rb = rb.pin_memory().to(decoder.device, non_blocking=True)
    return rb, len(starts)


class GraphedDecodeMixin:
    """decode_step(): a step of one row per request, captured once per (rows, cache) and replayed. Every kernel of such a step
    takes positions and slots from device memory and no launch shape depends on the contexts' lengths, so one capture serves
    while the requests grow."""

    class _Graph:
        pass

    def _init_graphs(self):
        self._graphs = {}         # (rows, id(cache)) -> captured decode-only step
        self.use_graph = True

    @torch.no_grad()
    def decode_step(self, meta_host: torch.Tensor, cache, max_keys: int) -> torch.Tensor:
        """meta_host int32 [3, B] (tokens, positions, slots; pinned host memory), one row per request. Returns fp32 logits
        [B, vocab] (a static buffer, overwritten by the next call)."""
        B = meta_host.shape[1]
        key = (B, id(cache))
        g = self._graphs.get(key)
        if g is not None and g.cache is not cache:
            g = None
        if g is None:
            if len(self._graphs) >= 16:
                self._graphs.pop(next(iter(self._graphs)))
            g = GraphedDecodeMixin._Graph()
            g.cache = cache
            g.meta = torch.zeros(3, B, device=self.device, dtype=torch.int32)
            g.want = torch.arange(B, device=self.device)
            g.graph = None
            self._graphs[key] = g
            if self.use_graph:
                # Capture needs a warmed-up step (kernel attributes, workspaces), but a step ADVANCES the per-slot states (a
                # convolution ring loses its oldest entry), so the warm-up must not touch live slots: it runs on a scratch cache
                # of the same shapes. The capture itself executes nothing.
                scratch = self.new_cache(2, cache.n_slots, 1)
                dummy = torch.zeros(3, B, device=self.device, dtype=torch.int32)
                dummy[2] = torch.arange(B, device=self.device, dtype=torch.int32) % cache.n_slots
                self.step(dummy[0], dummy[1], dummy[2], scratch, g.want, one_row_each=True)
                torch.cuda.synchronize()
                del scratch, dummy
                n0 = lib.launch_count()
                g.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g.graph):
                    g.logits = self.step(g.meta[0], g.meta[1], g.meta[2], cache, g.want, one_row_each=True)
                g.launches = lib.launch_count() - n0
                lib.add_launches(-g.launches)   # the capture does not execute
        g.meta.copy_(meta_host, non_blocking=True)
        if g.graph is None:
            return self.step(g.meta[0], g.meta[1], g.meta[2], cache, g.want, one_row_each=True)
        g.graph.replay()
        lib.add_launches(g.launches)
        return g.logits


class SequenceStepLM:
    """Entry point of a sequence-step model: from_pretrained / from_state_dict, step() for serving loops, generate() for greedy
    generation."""
    config_class = None
    decoder_class = None
    weights_from_state_dict = None

    def __init__(self, config, weights, dtype: torch.dtype = torch.bfloat16):
        if not torch.cuda.is_available():
            raise lib.OmcError("omchat_b200 needs a CUDA device (sm_100a); there is no CPU fallback")
        seqlib.load()
        self.config, self.weights, self.dtype = config, weights, dtype
        self.device = weights.embed.device
        self.decoder = self.decoder_class(config, weights, dtype)
        self.vocab_size = config.vocab_size

    @classmethod
    def from_state_dict(cls, sd, config, device="cuda", dtype: torch.dtype = torch.bfloat16, **unused):
        if not torch.cuda.is_available():
            raise lib.OmcError("omchat_b200 needs a CUDA device (sm_100a); there is no CPU fallback")
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("compute dtype must be torch.bfloat16 or torch.float32")
        device = torch.device(device)
        if device.type == "cuda" and device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        return cls(config, cls.weights_from_state_dict(sd, config, device, dtype), dtype)

    @classmethod
    def from_pretrained(cls, path: str, config=None, device="cuda", dtype: torch.dtype = torch.bfloat16, **kw):
        from .checkpoint import load_checkpoint
        sd, cfg = load_checkpoint(path, config)
        if not isinstance(cfg, cls.config_class):
            raise ValueError(f"{path} is not a {cls.config_class.__name__.replace('Config', '')} checkpoint")
        return cls.from_state_dict(sd, cfg, device=device, dtype=dtype)

    def eval(self):
        return self

    def step(self, tokens, pos, slot, cache, want_rows=None, collect=None, portions=None):
        with torch.cuda.device(self.device):
            return self.decoder.step(tokens, pos, slot, cache, want_rows, collect, portions)

    def decode_step(self, meta_host, cache, max_keys: int):
        """Decode-only batch (one token per request) through the captured CUDA graph; see GraphedDecodeMixin.decode_step."""
        with torch.cuda.device(self.device):
            return self.decoder.decode_step(meta_host, cache, max_keys)

    @torch.no_grad()
    def generate(self, input_ids, max_new_tokens: int = 32, eos_token_id: Optional[int] = None, do_sample: bool = False,
                 slots: int = 4, chunk: int = 512, **unused) -> List[torch.Tensor]:
        """Greedy generation of a batch of prompts (a [b, S] tensor or a list of 1-D id sequences of unequal length) through
        serving.StepScheduler: prompts are prefilled in portions of `chunk` tokens beside the decode rows of the requests that
        are already generating. Returns one LongTensor per prompt: the prompt followed by the generated ids."""
        if do_sample:
            raise NotImplementedError("only greedy decoding (do_sample=False) is on the accelerated path")
        from ..serving import StepScheduler
        prompts = [torch.as_tensor(p).view(-1).tolist() for p in input_ids]
        ps = self.config.kv_page_size
        need = sorted((-(-(len(p) + max_new_tokens) // ps) * ps for p in prompts), reverse=True)
        sched = StepScheduler(self, max_tokens=sum(need[:slots]), slots=slots, chunk=chunk)
        eos = self.config.eos_token_id if eos_token_id is None else eos_token_id
        rids = [sched.submit(p, max_new_tokens, eos) for p in prompts]
        res = sched.run()
        return [torch.tensor(p + res[r], dtype=torch.int64) for p, r in zip(prompts, rids)]
