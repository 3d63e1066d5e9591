"""The device timeline: the kernel libraries' traced build notes, per CTA, when a kernel was entered and when
its wait on the kernel before it was over.  Run in a process of its own (the traced build has to be chosen
before the first library is loaded): a tiny model decodes a few steps and the records are read back."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = textwrap.dedent("""
    import sys, tempfile
    sys.path.insert(0, {root!r}); sys.path.insert(0, {root!r} + "/tests")
    from kappai_b200.ops import timeline, build
    timeline.enable()
    import torch
    from kappai_b200 import ModelRunner, StepEntry, write_random_model
    from kappai_b200.ops import kernels as K
    from kappai_b200.sampling.sampler import argmax
    from tiny_configs import TINY_A, TINY_A_SEED
    with tempfile.TemporaryDirectory() as d:
        write_random_model(TINY_A, d, TINY_A_SEED)
        r = ModelRunner(d, dtype="bfloat16", max_tokens=256, max_requests=2, page_size=16)
        tok = argmax(r.step([StepEntry("a", [1, 2, 3, 4, 5], [4])]))
        timeline.records()
        K.LAUNCH_LOG[0] = []
        logits = r.step([StepEntry("a", [0], [0])], device_tokens=tok)
        names = list(K.LAUNCH_LOG[0]); K.LAUNCH_LOG[0] = None
        torch.cuda.synchronize()
        rec = timeline.records()
        ks = timeline.kernels(rec)
        # (a launcher may start more than one kernel: the scalar split-KV attention starts its merge itself)
        assert len(rec) > 0 and len(names) <= len(ks) <= 2 * len(names), (len(rec), len(ks), len(names))
        assert all("timeline" in k or "." not in k for k in build.loaded_libraries())
        last = None
        for k in ks:
            assert k["waited_first"] is not None and k["waited_first"] >= k["entered"] - 1e-3, k
            assert last is None or k["waited_first"] >= last - 1e-3, "a kernel's wait ended before its predecessor's"
            last = k["waited_first"]
        assert len(timeline.records()) == 0, "reading the records clears them"
        print(timeline.table(ks).splitlines()[1])
        print("timeline ok", len(ks))
    """)


def test_a_decode_step_leaves_a_mark_for_every_launch(tmp_path):
    p = subprocess.run([sys.executable, "-c", SCRIPT.format(root=ROOT)], capture_output=True, text=True, timeout=900)
    assert p.returncode == 0 and "timeline ok" in p.stdout, p.stdout[-2000:] + p.stderr[-4000:]
