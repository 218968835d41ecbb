"""The oracle's functional decoder against logits produced by the reference's own module code."""
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from oracle.model import OracleExecutor, OracleModel

GOLD = Path(__file__).parent / "golden"

QCFG = SimpleNamespace(hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                       num_hidden_layers=2, intermediate_size=128, vocab_size=211, rms_norm_eps=1e-6,
                       rope_theta=1e6, max_position_embeddings=1024)
GCFG = SimpleNamespace(hidden_size=64, num_attention_heads=4, num_key_value_heads=1, head_dim=32,
                       num_hidden_layers=6, intermediate_size=128, vocab_size=211, rms_norm_eps=1e-6,
                       rope_theta=1e6, rope_local_base_freq=1e4, query_pre_attn_scalar=32, sliding_window=512,
                       max_position_embeddings=1024)


@pytest.mark.parametrize("family,cfg,fname", [("qwen3", QCFG, "qwen3_tiny.npz"), ("gemma3", GCFG, "gemma3_tiny.npz")])
def test_tiny_model_logits_match_reference_modules(family, cfg, fname):
    z = np.load(GOLD / fname)
    weights = {k[2:]: torch.from_numpy(z[k]).to(torch.bfloat16) for k in z.files if k.startswith("w/")}
    weights = {k: (v.float() if "cos_sin" in k else v) for k, v in weights.items()}
    model = OracleModel(weights, cfg, family, num_blocks=8, block_size=256)
    ex = OracleExecutor(model, 256)
    lens, nblk = z["lens"].tolist(), z["nblocks"].tolist()
    toks, blks, ct, cb = [], [], 0, 0
    for n, nb in zip(lens, nblk):
        toks.append(z["tokens_flat"][ct:ct + n].tolist()); ct += n
        blks.append(z["blocks_flat"][cb:cb + nb].tolist()); cb += nb
    reqs = [SimpleNamespace(tokens=t, blocks=b, num_cached_tokens=0) for t, b in zip(toks, blks)]

    def logits_of(batch_type):
        from oracle import packing
        if batch_type == 0:
            p = packing.build_prefill_input([r.tokens for r in reqs], [r.blocks for r in reqs], [0] * len(reqs), 256)
        else:
            p = packing.build_decode_input([r.tokens for r in reqs], [r.blocks for r in reqs], 256)
        t = lambda a: None if a is None else torch.from_numpy(a)
        ctx = {"prefill": batch_type == 0, "slot_mapping": t(p["slot_mapping"]), "block_table": t(p["block_table"]),
               "cu_seqlens_q": t(p.get("cu_seqlens_q")), "cu_seqlens_k": t(p.get("cu_seqlens_k")),
               "cache_seqlens": t(p.get("cache_seqlens"))}
        return model.forward(ctx, t(p["input_ids"]), t(p["positions"])).float()

    got = logits_of(0)
    want = torch.from_numpy(z["prefill_logits"])
    # bf16 CPU GEMMs may pick different kernels on another host: compare with a bf16-sized tolerance
    assert (got - want).abs().max().item() <= 0.05 * max(1.0, want.abs().max().item())
    assert (got.argmax(-1) == want.argmax(-1)).all()
    for step in range(3):
        nxt = want.argmax(-1).tolist()
        for r, tok in zip(reqs, nxt):
            r.tokens.append(tok)
        got = logits_of(1)
        want = torch.from_numpy(z["decode_logits"][step])
        assert (got - want).abs().max().item() <= 0.05 * max(1.0, want.abs().max().item())
