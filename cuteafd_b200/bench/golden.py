"""``cuteafd golden``: layer-by-layer comparison of the CUDA engine against the CPU oracle on the
same weights and tokens; writes tokens / per-layer residual / logits statistics.

Counterpart: python/reference/layer_major.py:1-22 and the per-family ``golden`` subcommands.
"""
from __future__ import annotations

import json


def run_golden(args) -> int:
    import torch

    from ..config import PRESETS, scaled_down
    from ..ref.model import KvState, RefDecoder, init_weights
    if args.snapshot:
        from ..loader.load import load_params
        cfg, params = load_params(args.snapshot)
    else:
        cfg = PRESETS[args.preset]()
        if cfg.num_layers > 4:
            cfg = scaled_down(cfg, layers=2)
        params = {k: v.to(torch.bfloat16).float() for k, v in init_weights(cfg, seed=0).items()}
    g = torch.Generator().manual_seed(1)
    tokens = torch.randint(0, cfg.vocab_size, (args.tokens,), generator=g)
    ref = RefDecoder(cfg, params)
    with torch.no_grad():
        ref_logits = ref.forward(tokens, KvState(cfg))
    report = {"model": cfg.name, "tokens": args.tokens, "oracle_top1": ref_logits.argmax(-1)[-8:].tolist()}
    if torch.cuda.is_available() and cfg.attention == "gqa":
        from ..models.gqa_moe import GqaMoeEngine, GqaMoeWeights, KvCache
        from ..runtime.generate import Generator
        from ..runtime.native import make_pool
        dev = torch.device("cuda:0")
        W = GqaMoeWeights.from_params(cfg, params, dev)
        pages = args.tokens // 64 + 4
        eng = GqaMoeEngine(cfg, W, KvCache(cfg, pages, dev), max_tokens=args.tokens, max_seqs=4)
        gen = Generator(eng, make_pool(pages), pages, 4, prefill_chunk=args.tokens, use_graphs=False)
        s = gen.table.new()
        gen.prefill(s, tokens.tolist())
        got = eng.logits[0].float().cpu()
        err = (got - ref_logits[-1]).abs().max().item()
        p, q = torch.log_softmax(ref_logits[-1], -1), torch.log_softmax(got, -1)
        report.update(engine_top1=int(got.argmax()), max_abs_err=err, kl=float((p.exp() * (p - q)).sum()),
                      top1_match=bool(got.argmax() == ref_logits[-1].argmax()))
    text = json.dumps(report, indent=1)
    if args.out:
        open(args.out, "w").write(text)
    print(text)
    return 0
