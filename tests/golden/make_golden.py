"""Make tests/golden/*.npz: logits of the reference's OWN model code for the tiny models.

Run once on a machine that has the reference checkout (no GPU needed):

    python tests/golden/make_golden.py /path/to/anticitoyen-vram

It writes a tiny Qwen3 folder with this package's random-weights mode, converts it
with the reference's ``convert_checkpoint`` in its bf16 (identity) format, loads it
with the reference's ``load_model(dtype=float32, device_override="cpu")`` and runs
the reference's ``ACVRamModel`` on one whole sequence with logits at every position
and no cache.  tests/test_plain.py compares the plain implementation with these
files; the weights are made again from the same seed there, and the .npz also keeps
a checksum of them.
"""

from __future__ import annotations

import contextlib
import io
import os
import sys
import tempfile

os.environ["CUDA_VISIBLE_DEVICES"] = ""
os.environ["ACVRAM_ECO"] = "off"
os.environ["ACVRAM_KV_FORMAT"] = "bf16"
os.environ["ACVRAM_REGIME_MUET"] = "1"

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import numpy as np  # noqa: E402
import torch  # noqa: E402


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    from acvram.engine.config import load_model_spec
    from acvram.engine.loader import load_model
    from acvram.engine.lot import ForwardBatch
    from acvram.hardware.profiles import load_profile
    from acvram.memory.tiering import PlannerOptions, auto_plan
    from acvram.quant.convert import ConversionOptions, convert_checkpoint

    from acvram_b200.weights import write_random_model
    from conftest import TINY_SEEDS, random_ids, tiny_config
    import plain_qwen3

    for name in ("A", "B"):
        cfg = tiny_config(name)
        folder = tempfile.mkdtemp(prefix=f"golden_{name}_")
        write_random_model(cfg, folder, TINY_SEEDS[name])
        spec = load_model_spec(folder, f"tiny{name}")
        plan, _ = auto_plan(spec, load_profile("rig-14900k-5090-3080ti"),
                            PlannerOptions(max_model_len=cfg.max_position_embeddings, max_concurrent_seqs=2,
                                           force_format="bf16"))
        out = tempfile.mkdtemp(prefix=f"golden_conv_{name}_")
        with contextlib.redirect_stdout(io.StringIO()):
            convert_checkpoint(folder, plan, ConversionOptions(out_dir=out), spec=spec)
            loaded = load_model(out, dtype=torch.float32, device_override="cpu",
                                max_model_len=cfg.max_position_embeddings)
        model = loaded.model
        model.caches = {}
        n = 33
        ids = torch.tensor(random_ids(cfg.vocab_size, n, seed=900 + TINY_SEEDS[name]))
        batch = ForwardBatch(tokens=ids, positions=torch.arange(n), seq_lens=[n], query_lens=[n],
                             block_tables=[torch.zeros(8, dtype=torch.long)], slot_mapping=torch.arange(n),
                             is_prefill=True)
        logits = model(batch, logits_positions=batch.all_token_indices()).float().numpy()
        _, tensors = plain_qwen3.read_folder(folder)
        checksum = float(sum(t.double().abs().sum() for t in tensors.values()))
        np.savez_compressed(os.path.join(HERE, f"tiny_{name}.npz"), ids=ids.numpy(), logits=logits.astype(np.float32),
                            weights_abs_sum=np.float64(checksum))
        mine = plain_qwen3.forward_logits(*plain_qwen3.read_folder(folder), ids.tolist()).numpy()
        print(f"tiny {name}: reference logits {logits.shape}, max |reference - plain| = {np.abs(logits - mine).max():.3e}")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <checkout of anticitoyun/anticitoyen-vram>")
    main(sys.argv[1])
