"""``python -m jax_llm_examples_b200.timeline --preset NAME [--layers L] --batch B --context C``: where the kernels of
one decode step lie on the GPU's clock.

The step is replayed from its CUDA graph, as in serving, with random weights and a cache filled to the context
length; the kernel libraries are built with ``-DJLX_TIMELINE`` (see ``tracing.DeviceTimeline``), into files of their
own beside the ordinary ones.  Output: one line per launch with the medians over ``--repeat`` recorded steps of

* ``at``: when the launch could start working (its wait for the predecessor ended), microseconds into the step;
* ``early``: how long before that its first block was already resident (programmatic dependent launch);
* ``busy``: from then to the exit of its last block;
* ``adds``: how much later it ended than everything before it, i.e. what it added to the step;
* marks: times of marked places inside the kernel (``JLX_TL_MARK`` in the sources), after ``at``.
"""

from __future__ import annotations

import os

import torch

from .tracing import TIMELINE_FLAG, DeviceTimeline


def main(argv=None) -> int:
    import argparse
    import random

    ap = argparse.ArgumentParser(description="device timeline of one decode step")
    ap.add_argument("--preset", default="scout16")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--steps", type=int, default=6, help="decode steps before the recorded ones")
    ap.add_argument("--repeat", type=int, default=9, help="recorded steps (the table shows medians)")
    ap.add_argument("--prompt", type=int, default=0, metavar="T",
                    help="instead of decode steps: steps of one T-token prompt portion each (run eagerly, as prompts are; "
                         "library kernels, which carry no stamps, show as gaps)")
    args = ap.parse_args(argv)
    extra = os.environ.get("JLX_B200_NVCC_EXTRA", "")
    if TIMELINE_FLAG not in extra.split():  # before the first kernel library is built or loaded
        os.environ["JLX_B200_NVCC_EXTRA"] = (extra + " " + TIMELINE_FLAG).strip()
    import jax_llm_examples_b200 as J

    cfg_json = J.preset(args.preset, num_hidden_layers=args.layers) if args.layers else J.preset(args.preset)
    model = J.random_model(cfg_json, seed=0, dtype="bfloat16")
    b = args.batch
    page = 64
    if args.prompt:
        return _prompt_steps(J, model, args, page)
    gen = J.Generator(model, max_tokens=b * (-(-args.context // page) * page), page_size=page, max_slots=b, max_tokens_per_step=max(b, 64),
                      max_seq_len=args.context)
    eng = gen.engine
    slots = [eng.new_request() for _ in range(b)]
    start_len = args.context - args.steps - args.repeat - 8
    for s in slots:
        eng.manager.reserve(s, start_len)
        eng.manager.commit(s, start_len)
    for t in eng.kv:
        t.normal_(0.0, 0.5)
    rng = random.Random(0)
    sampler = J.Sampler(0)
    timeline = DeviceTimeline()

    def one_step():
        logits = eng.step([J.StepEntry(s, [rng.randrange(model.config.vocab_size)], [0]) for s in slots])
        return sampler.sample(logits, [0.0] * b, [0] * b, [0] * b, [0] * b)

    for _ in range(args.steps):
        one_step()
        timeline.attach()
    recorded = []
    for _ in range(args.repeat):
        torch.cuda.synchronize()
        timeline.reset()
        one_step()
        recorded.append(timeline.launches())
    eng.check_status()
    rows = DeviceTimeline.summary(recorded)
    print(f"# one decode step, {args.preset}, {model.config.num_hidden_layers} layers, batch {b}, context {args.context}: "
          f"{len(rows)} launches, {sum(r['adds'] for r in rows):.1f} us (medians of {args.repeat} steps, in us)")
    print(DeviceTimeline.table(rows))
    return 0


def _prompt_steps(J, model, args, page) -> int:
    import random

    T = args.prompt
    rng = random.Random(0)
    gen = J.Generator(model, max_tokens=(args.steps + args.repeat + 1) * (-(-T // page) * page), page_size=page,
                      max_slots=args.steps + args.repeat + 1, max_tokens_per_step=T, max_seq_len=max(T, page))
    eng = gen.engine
    timeline = DeviceTimeline(capacity=1 << 18)

    def one_step():
        s = eng.new_request()
        eng.step([J.StepEntry(s, [rng.randrange(model.config.vocab_size) for _ in range(T)], [T - 1])])
        torch.cuda.synchronize()
        eng.finish(s)

    for _ in range(args.steps):
        one_step()
        timeline.attach()
    recorded = []
    for _ in range(args.repeat):
        timeline.reset()
        one_step()
        recorded.append(timeline.launches())
    eng.check_status()
    rows = DeviceTimeline.summary(recorded)
    print(f"# one step of a {T}-token prompt, {args.preset}, {model.config.num_hidden_layers} layers: {len(rows)} stamped launches "
          f"(medians of {args.repeat} steps, in us)")
    print(DeviceTimeline.table(rows))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
