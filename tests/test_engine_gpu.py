"""The engine against the plain implementation, in 32-bit and in bfloat16,
under every way of cutting the work."""
import numpy as np
import pytest
import torch

from helpers import TINY, TOL, make_folder, plain_logits, random_ids, rel_err

pytestmark = pytest.mark.gpu


def _engine(folder, dtype, n_pages=64, page_size=16, **kw):
    from gibbs_b200 import Engine, load_model
    model = load_model(folder, dtype=dtype, device="cuda:0")
    return Engine(model, n_pages=n_pages, page_size=page_size, **kw)


def _stored(dtype):
    return torch.bfloat16 if dtype == "bfloat16" else torch.float32


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_prompt(tmp_path, name, dtype):
    from gibbs_b200 import StepEntry
    folder = make_folder(tmp_path, name, stored=_stored(dtype))
    eng = _engine(folder, dtype)
    vocab = TINY[name][0]["vocab_size"]
    for seed, n in ((1, 1), (2, 7), (3, 40), (4, 150)):
        ids = random_ids(seed, n, vocab)
        eng.open("r")
        got = eng.step([StepEntry("r", ids, list(range(n)))]).cpu().numpy()
        eng.check_status()
        eng.close("r")
        want = plain_logits(folder, ids)
        assert got.shape == want.shape
        assert rel_err(got, want) < TOL[dtype], (n, rel_err(got, want))
    eng.cache.check()
