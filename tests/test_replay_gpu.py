"""bin/trace_run as a user runs it: a subprocess, steps on standard input one at a time (the next only after
`done <step>`), logits from the files it writes, in 32-bit and in bfloat16, against the plain implementation."""

import json
import random
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _replay(model_dir, dtype, steps, out_dir, max_tokens, vocab, extra=()):
    cmd = [sys.executable, str(Path(H.ROOT) / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(max_tokens), *extra]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    got, at = {}, {}
    try:
        for i, st in enumerate(steps):
            proc.stdin.write(json.dumps({"step": i, **st}) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {i}", (line, proc.stderr.read()[-3000:] if proc.poll() is not None else "")
            places = []
            for e in st["entries"]:
                places += [(e["id"], at.get(e["id"], 0) + w) for w in e["want"]]
                at[e["id"]] = at.get(e["id"], 0) + len(e["tokens"])
            path = Path(out_dir) / f"{i}.f32"
            if places:
                rows = np.fromfile(path, dtype="<f4").reshape(len(places), vocab)
                for key, row in zip(places, rows):
                    got[key] = row
            else:
                assert not path.exists()
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    return got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_replays_mixed_steps_with_reused_pages(model_dirs, tmp_path, dtype):
    rng = random.Random(12)
    lengths = [120, 64, 65, 3, 100, 130, 31, 90]
    reqs = H.random_requests(rng, 384, lengths)
    steps = H.trace_mixed(reqs, rng, max_live=4)
    steps.insert(3, {"entries": [], "end": []})  # a step with nothing in it is answered too
    # 4 live requests of at most 130 tokens, each rounded up to 64: 4 * 192 tokens; 8 requests need far more in total
    got = _replay(model_dirs["tiny_b"], dtype, steps, tmp_path / "out", 4 * 192, 384)
    assert len(got) == sum(lengths)
    worst = 0.0
    for rid, toks in reqs.items():
        ref, _ = H.plain_logits(model_dirs["tiny_b"], toks)
        errs = [H.rel_err(got[(rid, p)], ref[p]) for p in range(len(toks))]
        if dtype == "float32":
            assert max(errs) < H.TOL[dtype], (rid, max(errs))
        else:
            # without the engine's expert choices a near-tie may flip a token's expert: most positions must
            # agree within the bfloat16 tolerance, and none may be far off
            assert np.mean(np.array(errs) < H.TOL[dtype]) > 0.9 and max(errs) < 0.5, (rid, max(errs))
        worst = max(worst, max(errs))
    print(f"trace_run {dtype}: worst relative error {worst:.2e}")


def test_trace_run_whole_then_one_by_one_agree_closely(model_dirs, tmp_path):
    rng = random.Random(3)
    reqs = H.random_requests(rng, 320, [150, 70])
    a = _replay(model_dirs["tiny_c"], "float32", H.trace_whole(reqs), tmp_path / "a", 256, 320)
    b = _replay(model_dirs["tiny_c"], "float32", H.trace_tail_decode(reqs, 32), tmp_path / "b", 256, 320)
    c = _replay(model_dirs["tiny_c"], "float32", H.trace_portions(reqs, rng), tmp_path / "c", 256, 320, ("--page-size", "16"))
    assert max(H.rel_err(b[k], a[k]) for k in a) < 2e-6 and max(H.rel_err(c[k], a[k]) for k in a) < 2e-6
    H.compare_plain_only(model_dirs["tiny_c"], reqs, a, "float32")
