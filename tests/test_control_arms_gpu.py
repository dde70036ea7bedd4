"""Arms that must break: a comparison with a tolerance proves something only if a fault of the kind it looks for
exceeds the tolerance (the reference builds its kernel tests the same way, tests/test_attn_paginee.py).  Here the
fault is a page of the wrong request in a block table (two live requests exchange one page between two steps): the
bfloat16 bound of the replay tests (2.5 times the plain implementation's own bfloat16-to-float32 distance) has to be
exceeded by it.  (Two pages of one request exchanged would prove nothing: keys are stored rotated, so the set of keys
and values that a later query sees is the same and only the order of the sum changes.)"""

from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_qwen3
from conftest import random_ids

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,dtype", [("F", "bfloat16"), ("D", "bfloat16"), ("A", "bfloat16"), ("F", "float32")])
def test_a_page_of_the_wrong_request_breaks_the_bound(name, dtype, tiny_folders, plain_models):
    from acvram_b200.engine.batch import StepEntry
    from acvram_b200.engine.runner import ModelRunner
    from acvram_b200.models import build_from_folder

    cfg, t = plain_models[name]
    run_dtype = getattr(torch, dtype)
    _, model = build_from_folder(tiny_folders[name], run_dtype)
    ids = random_ids(cfg["vocab_size"], 200, 41)
    other = random_ids(cfg["vocab_size"], 64, 42)
    ref = plain_qwen3.forward_logits(cfg, t, ids).numpy()
    if dtype == "bfloat16":
        bound = 2.5 * float(np.abs(plain_qwen3.forward_logits(cfg, t, ids, torch.bfloat16).numpy() - ref).max())
    else:
        bound = 2e-5 * max(1.0, float(np.abs(ref).max()))

    def tail_distance(exchange: bool) -> float:
        runner = ModelRunner(model, 16, 32, 2)
        if run_dtype == torch.bfloat16:
            runner.enable_graphs()
        runner.step([StepEntry("r", ids[:192], ())])
        runner.step([StepEntry("s", other, ())])
        if exchange:
            group = runner.manager.paged_groups[0]
            mine, theirs = group.tables["r"][11], group.tables["s"][3]
            group.set_page("r", 11, theirs)
            group.set_page("s", 3, mine)
        worst = 0.0
        for i in range(192, 200):
            lg = runner.step([StepEntry("r", ids[i:i + 1], (0,))])
            worst = max(worst, float(np.abs(lg[0].float().cpu().numpy() - ref[i]).max()))
        runner.check_status()
        runner.release("r")
        runner.release("s")
        runner.manager.check()
        return worst

    good, bad = tail_distance(False), tail_distance(True)
    assert good <= bound, f"the unchanged arm is off by {good:.3e} (bound {bound:.3e})"
    assert bad > bound, f"a wrong page moves the logits by only {bad:.3e}; the bound {bound:.3e} would not see it"
