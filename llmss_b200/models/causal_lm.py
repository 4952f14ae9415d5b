"""HF-shaped entry points: ``MODEL_REGISTRY[model_type](config, weights)``.

Parity with the reference's constructor / forward contract (gptj_modeling.py:517-634,
gpt_bigcode_modeling.py:786-915): ``model(input_ids, past_key_values=None, use_cache=None)``
returns an object with ``.logits`` ([B, S, V] fp32) and ``.past_key_values``.  The cache
object is an opaque :class:`PagedState` (pre-allocated paged KV, no per-step torch.cat),
which callers simply pass back, exactly as generate.py:104-106 does with HF tuples.
The serving engine does not use this wrapper; it drives ``.core`` (DecoderLM) directly.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
from torch import nn

from ..engine.batch import BatchInput
from .bedovik import BedovikLM, bedovik_spec, load_bedovik
from .botalorn import BotalornLM, botalorn_spec, load_botalorn
from .decoder import DecoderLM
from .families import FAMILIES
from .ninelix import NinelixLM, load_ninelix, ninelix_spec
from .zenorax import ZenoraxLM, load_zenorax, zenorax_spec


class PagedState:
    """KV state of a fixed set of B sequences advancing in lock-step (HF-compat path)."""

    def __init__(self, core: DecoderLM, batch_size: int, capacity: int, block_size: int = 16):
        self.core, self.B, self.block_size = core, batch_size, block_size
        self.length = 0
        self._alloc(capacity)

    def _alloc(self, capacity: int):
        bs = self.block_size
        self.blocks_per_seq = max(1, -(-capacity // bs))
        self.capacity = self.blocks_per_seq * bs
        self.kv = self.core.make_cache(1 + self.B * self.blocks_per_seq, bs, max_seqs=self.B)   # sequence i keeps state slot i
        self.tables = [[1 + i * self.blocks_per_seq + j for j in range(self.blocks_per_seq)] for i in range(self.B)]

    def ensure(self, total_len: int):
        if total_len <= self.capacity:
            return
        old_kv, old_bps = self.kv, self.blocks_per_seq
        self._alloc(max(total_len, 2 * self.capacity))
        # copy the live blocks of every sequence (and, with them, the state slots) into the enlarged cache
        for i in range(self.B):
            src = 1 + i * old_bps
            dst = 1 + i * self.blocks_per_seq
            self.kv.copy_blocks_from(old_kv, src, dst, old_bps)

    def get_seq_length(self) -> int:
        return self.length


@dataclass
class CausalLMOutputWithPast:
    logits: torch.Tensor
    past_key_values: Optional[PagedState] = None
    loss: Optional[torch.Tensor] = None

    def __getitem__(self, i):
        return (self.logits, self.past_key_values)[i]


class CausalLM(nn.Module):
    family: str = ""
    float32_on_cuda: bool = False   # the multi-head families' CUDA kernels take 16-bit activations only

    def __init__(self, config, weights, fuse_parallel: bool = True):
        super().__init__()
        spec_fn, load_fn = FAMILIES[self.family]
        self.config = config
        self.core = DecoderLM(spec_fn(config), weights.process_group, weights.device, weights.dtype,
                              fuse_parallel=fuse_parallel)
        load_fn(self.core, weights)
        self.core.finalize()

    @property
    def spec(self):
        return self.core.spec

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, past_key_values: Optional[PagedState] = None,
                use_cache: Optional[bool] = None, last_only: bool = False, **_unused) -> CausalLMOutputWithPast:
        core = self.core
        B, S = input_ids.shape
        st = past_key_values
        if st is None:
            st = PagedState(core, B, capacity=min(core.spec.max_pos, S + 64))
        assert st.B == B, "batch size changed between calls"
        ctx = st.length
        st.ensure(ctx + S)
        ids = input_ids.tolist()
        batch = BatchInput.build(ids, [ctx] * B, st.tables, st.block_size, core.device, max_blocks=st.blocks_per_seq,
                                 state_slots=list(range(B)) if getattr(core, "needs_state", False) else None)
        hidden = core.forward_hidden(batch, st.kv)
        if last_only:
            logits = core.logits(hidden.index_select(0, batch.last_idx))[:, :core.spec.vocab].reshape(B, 1, -1)
        else:
            logits = core.logits(hidden)[:, :core.spec.vocab].reshape(B, S, -1)
        st.length = ctx + S
        return CausalLMOutputWithPast(logits=logits.float(), past_key_values=st if use_cache else None)


class GPTJForCausalLM(CausalLM):
    family = "gptj"


class GPTBigCodeForCausalLM(CausalLM):
    family = "gpt_bigcode"


class GPT2LMHeadModel(CausalLM):
    family = "gpt2"


class OPTForCausalLM(CausalLM):
    family = "opt"


class LlamaForCausalLM(CausalLM):
    family = "llama"


class BedovikForCausalLM(CausalLM):
    """Native architecture (config.json with an ``architecture`` key, see models/bedovik.py): latent attention, routed
    experts, Dynamic Tanh, weight-shared loop.  Same constructor and forward interface as the HF-shaped classes."""
    family = "bedovik"
    float32_on_cuda = True          # every kernel of this family also exists in true 32-bit

    def __init__(self, config, weights, fuse_parallel: bool = True):
        nn.Module.__init__(self)
        self.config = config
        self.core = BedovikLM(bedovik_spec(config), weights.process_group, weights.device, weights.dtype)
        load_bedovik(self.core, weights)
        self.core.finalize()


class NinelixForCausalLM(CausalLM):
    """Native architecture (see models/ninelix.py): recurrent mixers and biased attention over a 32-bit residual stream
    with post-normed sub-layers.  Same constructor and forward interface as the HF-shaped classes."""
    family = "ninelix"
    float32_on_cuda = True

    def __init__(self, config, weights, fuse_parallel: bool = True):
        nn.Module.__init__(self)
        self.config = config
        self.core = NinelixLM(ninelix_spec(config), weights.process_group, weights.device, weights.dtype)
        load_ninelix(self.core, weights)
        self.core.finalize()


class BotalornForCausalLM(CausalLM):
    """Native architecture (see models/botalorn.py): hyper-connected residual streams, sliding-window attention with
    shared keys / values, gated delta rule.  Same constructor and forward interface as the HF-shaped classes."""
    family = "botalorn"
    float32_on_cuda = True

    def __init__(self, config, weights, fuse_parallel: bool = True):
        nn.Module.__init__(self)
        self.config = config
        self.core = BotalornLM(botalorn_spec(config), weights.process_group, weights.device, weights.dtype)
        load_botalorn(self.core, weights)
        self.core.finalize()


class ZenoraxForCausalLM(CausalLM):
    """Native architecture (see models/zenorax.py): sub-layers normed on both sides, input convolutions, depth-weighted
    averaging of layer outputs, latent attention with a rotated key part, sink attention, a gated linear recurrence.  Same
    constructor and forward interface as the HF-shaped classes."""
    family = "zenorax"
    float32_on_cuda = True

    def __init__(self, config, weights, fuse_parallel: bool = True):
        nn.Module.__init__(self)
        self.config = config
        self.core = ZenoraxLM(zenorax_spec(config), weights.process_group, weights.device, weights.dtype)
        load_zenorax(self.core, weights)
        self.core.finalize()


MODEL_REGISTRY = {
    "gptj": GPTJForCausalLM,
    "gpt_bigcode": GPTBigCodeForCausalLM,
    "gpt2": GPT2LMHeadModel,
    "opt": OPTForCausalLM,
    "llama": LlamaForCausalLM,
    "bedovik": BedovikForCausalLM,
    "ninelix": NinelixForCausalLM,
    "botalorn": BotalornForCausalLM,
    "zenorax": ZenoraxForCausalLM,
}
