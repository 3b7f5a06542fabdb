"""Developer CLI: ``python -m megabake_b200 {decode,prefill} --mode ...`` runs a seeded
synthetic decoder through ``make_backend`` (the reference's ``--mode prefill|decode``,
``--fallback`` and ``--no-cache`` flags, src/megabake/main.py:221-231)."""

from __future__ import annotations

import argparse
import time

import torch


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="megabake_b200")
    parser.add_argument("command", choices=["decode", "prefill"])
    parser.add_argument("--mode", choices=["prefill", "decode"], default=None,
                        help="backend mode policy (defaults to the command)")
    parser.add_argument("--fallback", choices=["error", "inductor"], default="error")
    parser.add_argument("--no-cache", action="store_true")
    parser.add_argument("--config", default="smollm-135m")
    parser.add_argument("--steps", type=int, default=8)
    parser.add_argument("--capacity", type=int, default=128)
    parser.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    parser.add_argument("--no-kernel", action="store_true", help="compile_kernel=False: run the captured graph")
    return parser


def main(argv=None) -> int:
    from transformers import LlamaConfig, LlamaForCausalLM, Qwen2Config, Qwen2ForCausalLM

    from . import CONFIGS, ExplicitStateDecoder, make_backend, register_transformers_attention
    from .synth import new_kv_state, synth_ids, synth_weights

    args = build_parser().parse_args(argv)
    config = CONFIGS[args.config]
    device = torch.device(args.device)
    common = dict(hidden_size=config.hidden, intermediate_size=config.intermediate,
                  num_attention_heads=config.q_heads, num_key_value_heads=config.kv_heads,
                  num_hidden_layers=config.layers, vocab_size=config.vocab, head_dim=config.head_dim,
                  max_position_embeddings=max(args.capacity, 16), rms_norm_eps=config.rms_eps,
                  tie_word_embeddings=config.tied,
                  rope_parameters={"rope_type": "default", "rope_theta": config.rope_theta})
    with torch.device("meta"):
        model = (Qwen2ForCausalLM(Qwen2Config(**common)) if config.qkv_bias else LlamaForCausalLM(LlamaConfig(**common)))
    model = model.to_empty(device=device).to(torch.bfloat16).eval()
    model.load_state_dict(synth_weights(config, seed=0, device=device), strict=False)
    model.model.rotary_emb.__init__(model.config, device=device)
    model.model.rotary_emb.to(torch.bfloat16)
    backend = make_backend(mode=args.mode or args.command, fallback=args.fallback, cache=not args.no_cache,
                           model_name=args.config, compile_kernel=False if args.no_kernel else None)
    ids = synth_ids(4, config.vocab, seed=0).to(device)
    with torch.no_grad():
        if args.command == "decode":
            step = torch.compile(ExplicitStateDecoder(model), backend=backend, fullgraph=True, dynamic=False)
            keys, values, lengths = new_kv_state(config, 1, args.capacity, device)
            state = [t for triple in zip(keys, values, lengths) for t in triple]
            token = ids[:1].view(1, 1)
            started = time.perf_counter()
            for position in range(args.steps):
                logits = step(token, torch.full((1, 1), position, dtype=torch.int64, device=device), *state)
                token = logits[:, 0].float().argmax(-1).view(1, 1)
            print(f"decoded {args.steps} tokens in {time.perf_counter() - started:.3f}s; last token {int(token)}")
        else:
            register_transformers_attention()
            model.set_attn_implementation("megabake")
            prompt = torch.compile(model, backend=backend, fullgraph=True, dynamic=False)
            logits = prompt(input_ids=ids.view(1, -1), use_cache=False).logits
            print(f"prefill logits {tuple(logits.shape)}; argmax of last position {int(logits[0, -1].float().argmax())}")
    print("execution:", backend.megabake_contexts[-1].requirements["execution"])
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
