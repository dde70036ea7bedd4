"""The reference arm of bench.py: the unmodified reference from baseline/_ref through its own public API.

What runs: the reference's ``load_model_spec`` -> ``detect_rig`` -> ``auto_plan`` -> ``convert_checkpoint``
(format bf16, an identity copy) -> ``load_model`` -> ``Engine.add_request`` / ``Engine.step``, on a model folder
with the sizes of Qwen3-8B and random weights that this file writes with plain torch and safetensors.  None of
acvram_b200's models, kernels or engine is on that path.  The metric is the one bench.py measures for its own
arm: decoded tokens per second of a batch of requests that each hold a context of synthetic tokens, over
exactly K steps after W warm-up steps, host token ids in and out.

When anything on the way cannot be had (no install, no CUDA device, an exception in the reference's code) one
line ``{"impl": "reference", "unavailable": "<why>"}`` is printed and the exit code is 0.
"""

from __future__ import annotations

import json
import os
import shutil
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


def unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:300]}))
    return 0


def write_model_folder(folder: str, cfg: dict, seed: int = 0) -> None:
    """config.json plus sharded safetensors, N(0, 0.02) matrices and norm weights 1 + N(0, 0.1), bfloat16."""
    import torch
    from safetensors.torch import save_file

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    gen = torch.Generator(device="cuda").manual_seed(seed)
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    NH, NKV, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]

    def mat(*shape):
        return (torch.randn(*shape, device="cuda", generator=gen) * 0.02).to(torch.bfloat16).cpu()

    def norm(n):
        return (1 + 0.1 * torch.randn(n, device="cuda", generator=gen)).to(torch.bfloat16).cpu()

    weight_map = {}

    def shard(name: str, tensors: dict) -> None:
        save_file(tensors, os.path.join(folder, name), metadata={"format": "pt"})
        weight_map.update({k: name for k in tensors})

    shard("model-embed.safetensors", {"model.embed_tokens.weight": mat(V, H), "model.norm.weight": norm(H)})
    shard("model-head.safetensors", {"lm_head.weight": mat(V, H)})
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        shard(f"model-layer{i}.safetensors", {
            p + "self_attn.q_proj.weight": mat(NH * D, H), p + "self_attn.k_proj.weight": mat(NKV * D, H),
            p + "self_attn.v_proj.weight": mat(NKV * D, H), p + "self_attn.o_proj.weight": mat(H, NH * D),
            p + "self_attn.q_norm.weight": norm(D), p + "self_attn.k_norm.weight": norm(D),
            p + "mlp.gate_proj.weight": mat(I, H), p + "mlp.up_proj.weight": mat(I, H),
            p + "mlp.down_proj.weight": mat(H, I), p + "input_layernorm.weight": norm(H),
            p + "post_attention_layernorm.weight": norm(H)})
    with open(os.path.join(folder, "model.safetensors.index.json"), "w") as fh:
        json.dump({"metadata": {}, "weight_map": weight_map}, fh)


def run(args) -> int:
    if not os.path.isdir(os.path.join(REF, "acvram")):
        return unavailable("baseline/_ref holds no install of the reference (pip install --no-deps --target baseline/_ref)")
    try:
        import torch
    except Exception as exc:  # noqa: BLE001
        return unavailable(f"torch cannot be imported: {exc}")
    if not torch.cuda.is_available():
        return unavailable("no CUDA device")

    os.environ.setdefault("ACVRAM_ECO", "off")            # never touch the clocks
    os.environ.setdefault("ACVRAM_KV_FORMAT", "bf16")      # the bf16 cache that the metric names
    os.environ.setdefault("ACVRAM_REGIME_MUET", "1")
    sys.path.insert(0, REF)
    work = tempfile.mkdtemp(prefix="acvram_ref_", dir=os.environ.get("ACVRAM_REF_TMP", tempfile.gettempdir()))
    try:
        from bench import SHAPES, bench_config  # the sizes and the configuration keys that bench.py names

        shape = SHAPES[getattr(args, "shape", "8b")]
        shape_name = f"Qwen3-{getattr(args, 'shape', '8b').upper()} shape"
        layers = args.layers or shape["num_hidden_layers"]
        cfg = {**shape, "num_hidden_layers": layers, "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
               "hidden_act": "silu", "torch_dtype": "bfloat16", "eos_token_id": 151645, "bos_token_id": 151643}
        hf = os.path.join(work, "hf")
        t0 = time.time()
        write_model_folder(hf, cfg)
        print(f"[reference arm] model folder written in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)

        from acvram.engine.config import load_model_spec
        from acvram.engine.loader import load_model
        from acvram.engine.runner import Engine
        from acvram.engine.sampler import SamplingParams
        from acvram.hardware.detect import detect_rig
        from acvram.memory.tiering import PlannerOptions, auto_plan
        from acvram.quant.convert import ConversionOptions, convert_checkpoint

        max_len = 8192
        spec = load_model_spec(hf, "qwen3-8b-shape")
        rig = detect_rig(None)
        plan, _ = auto_plan(spec, rig, PlannerOptions(max_model_len=max_len, max_concurrent_seqs=args.batch,
                                                      force_format="bf16"))
        conv = os.path.join(work, "converted")
        t0 = time.time()
        convert_checkpoint(hf, plan, ConversionOptions(out_dir=conv), spec=spec)
        shutil.rmtree(hf, ignore_errors=True)
        print(f"[reference arm] converted in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
        loaded = load_model(conv, max_model_len=max_len, max_concurrent_seqs=args.batch)
        engine = Engine(loaded, None, max_batch_size=args.batch, max_model_len=max_len)

        K, W = args.steps, max(3, args.warmup)
        vocab = cfg["vocab_size"]
        params = SamplingParams(temperature=0.0, max_tokens=K + W + 8, ignore_eos=True)
        for k in range(args.batch):
            prompt = [((50 + k) * 104729 + i * 7919) % (vocab - 100) + 10 for i in range(args.context)]
            engine.add_request(prompt, params)
        # run until every request has its prompt behind it and decodes
        guard = 0
        produced = 0
        while produced < args.batch and guard < 10000:
            produced += sum(1 for o in engine.step() if o.token_ids)
            guard += 1
        for _ in range(W):
            engine.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        tokens = 0
        for _ in range(K):
            tokens += sum(len(o.token_ids) for o in engine.step())
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        line = {"impl": "reference", "metric": f"decode tok/s at batch {args.batch} ({shape_name}, {args.context}-token contexts)",
                "value": round(tokens / dt, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
                "ms_per_step": round(dt / K * 1e3, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic token ids, random weights N(0,0.02)",
                # the same keys and, where they describe the workload, the same values as the other arm's line; the
                # reference's page is 16 tokens, fixed in its code, and it times with the wall clock around Engine.step
                "config": bench_config(args, cfg, layers, shape["num_hidden_layers"], 16, True),
                "e2e": {"value": round(tokens / dt, 1), "unit": "tokens/s"}}
        print(json.dumps(line))
        return 0
    except BaseException as exc:  # noqa: BLE001  (the reference may call sys.exit)
        if isinstance(exc, KeyboardInterrupt):
            raise
        return unavailable(f"the reference failed on this box: {type(exc).__name__}: {exc}")
    finally:
        shutil.rmtree(work, ignore_errors=True)
