"""Every script under examples/ runs to completion on CPU."""
import os
import runpy

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPTS = sorted(
    os.path.join(d, f)[len(ROOT) + 1:]
    for d, _, fs in os.walk(os.path.join(ROOT, "examples")) for f in fs if f.endswith(".py"))


@pytest.mark.parametrize("script", SCRIPTS)
def test_example_runs(script, tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    torch.manual_seed(0)
    ns = runpy.run_path(os.path.join(ROOT, script), run_name="example")
    main = ns["main"]
    if script.endswith("train_gpt2_sharded.py"):
        if torch.cuda.is_available():
            pytest.skip("covered by the GPU tests")
        out = main(["--steps", "2"])
        assert len(out) == 2 and all(v == v for v in out)
    elif "train_" in script:
        losses = main()
        assert all(v == v for v in losses)
        if "cnn" not in script:
            assert losses[-1] < losses[0]
    else:
        assert main() is not None
