"""The engine-facing half of the reference's vLLM model class `BitExactLlamaForCausalLM`
(src/bitexact/vllm_plugin/model.py:63-357): what happens between vLLM's calls and the integer engine.

`ModelGlue` holds an engine of this package (`ExactEngine` / `IntEngine`) and provides, with the reference's
behaviour:

  embed_input_ids(ids)                       the integer embedding rows (model.py:146-147)
  forward(ids, positions, meta, kv_caches)   any mix of decode and prompt tokens as rows with their request's
                                             block-table row (`_forward_exact`, model.py:259-288): `meta` is vLLM's
                                             attention metadata (query_start_loc, seq_lens, slot_mapping,
                                             block_table); padding rows go to the null block
  compute_logits(hidden_states)              integer logits -> STASH for the sampler + the float rows vLLM wants
                                             (model.py:300-317): real floats only for strict requests, one-hot rows
                                             at the greedy token otherwise, an uninitialised buffer when the
                                             sampler's noisy pass rewrites every row anyway
  check_late() / check_output()              the bound flag without a host sync: copied to pinned memory each step,
                                             read when the step's output is collected (model.py:290-298)

What stays with the maintainer's vLLM-side class: registering the architecture, the `Attention` layers that make
vLLM allocate the paged cache (HKV heads of 2 HD bf16 = 8 HD bytes per token, reinterpreted as limb planes), and
handing `get_forward_context().attn_metadata` and the layers' `kv_cache` tensors to `forward`."""

import torch

from . import tri_logits
from .sampler import STASH


class ModelGlue:
    def __init__(self, engine, spec_q=1):
        self.m = engine
        self.exact = engine.FR == 24
        self.spec_q = spec_q                                      # query tokens per request in a decode step
        self.qdim = engine.H * engine.HD
        self.flag = torch.zeros((), dtype=torch.bool, device="cpu",
                                pin_memory=torch.cuda.is_available())
        STASH.active, STASH.lnt, STASH.fr = True, engine.ln, engine.FR

    def embed_input_ids(self, input_ids):
        return self.m.emb[input_ids].long()

    def rows(self, positions, meta, N):
        """-> (pos, slot, rmap, n): per token row its position, cache slot (-1: padding) and block-table row; n rows
        are real. One host read of query_start_loc (vLLM keeps a host copy)."""
        qsl = [int(v) for v in meta.query_start_loc.cpu().tolist()]
        R = len(meta.seq_lens)
        n = min(qsl[R], N)
        dev = positions.device
        if n == N == R and self.spec_q == 1:                      # uniform decode: row r belongs to request r
            return positions, meta.slot_mapping[:N], torch.arange(N, device=dev), n
        counts = torch.tensor([qsl[r + 1] - qsl[r] for r in range(R)])
        rmap = torch.zeros(N, dtype=torch.long)
        rmap[:n] = torch.repeat_interleave(torch.arange(R), counts)[:n]
        slot = torch.full((N,), -1, dtype=torch.long, device=dev)
        slot[:n] = meta.slot_mapping[:n]
        pos = positions.clone()
        pos[n:] = 0
        return pos, slot, rmap.to(dev), n

    def forward(self, input_ids, positions, meta, kv_caches):
        """-> the residual stream int64 [N, D] (vLLM's hidden states)."""
        N = input_ids.shape[0]
        pos, slot, rmap, _ = self.rows(positions, meta, N)
        return self.m.forward(kv_caches, input_ids, pos, slot, meta.block_table, rmap)

    def check_late(self):
        self.flag.copy_(self.m.fl[0] != 0, non_blocking=True)

    def check_output(self):
        """Call after the step's outputs have reached the host (vLLM's own wait covers the copy)."""
        if bool(self.flag):
            raise OverflowError("integer bound violated")

    def compute_logits(self, hidden_states):
        mm = self.m
        li = mm.logits(hidden_states.long())
        self.check_late()
        STASH.head, STASH.logits = None, li
        smp = STASH.sampler
        STASH.strict = smp is None or smp.any_strict()
        if not STASH.strict and smp.any_noisy():
            # temperature rows: the sampler's pass chooses every token (greedy rows too) and rewrites all rows
            _, STASH.greedy = tri_logits.argmax_float(li, mode="none")
            return torch.empty(li.shape, dtype=torch.float32, device=li.device)
        f, STASH.greedy = tri_logits.argmax_float(li, scale=2.0 ** -mm.FR, mode="float" if STASH.strict else "onehot")
        return f

    def load_weights(self, weights):
        for _ in weights:                                         # the integer constants were loaded with the engine
            pass
        return set()
