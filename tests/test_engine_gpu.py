"""The engine against the plain implementation, on a GPU, in 32-bit and in bfloat16: the same
requests whole; most of each in one step and the last 32 tokens one by one; in portions of changing
size; and mixed, with so few pages that they are used again."""

import random

import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu

LENGTHS = {"tiny_a": [80, 1, 33, 47, 64, 17], "tiny_b": [130, 49, 2, 97, 48, 75], "tiny_c": [200, 81, 3, 160, 65, 129]}
VOCAB = {"tiny_a": 256, "tiny_b": 384, "tiny_c": 320}
NAMES = ["tiny_a", "tiny_b", "tiny_c"]


def _engine(model_dir, dtype, max_tokens, page_size=16, max_slots=8):
    import jax_llm_examples_b200 as J

    model = J.load_model(model_dir, dtype, "cuda")
    return J.Engine(model, max_tokens=max_tokens, page_size=page_size, max_slots=max_slots)


def _requests(name, seed=0):
    return H.random_requests(random.Random(seed), VOCAB[name], LENGTHS[name])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_whole_requests(model_dirs, name, dtype):
    reqs = _requests(name)
    eng = _engine(model_dirs[name], dtype, max_tokens=208)
    got, routing = H.run_trace(eng, H.trace_whole(reqs))
    worst = H.compare_with_plain(model_dirs[name], reqs, got, routing, dtype)
    print(f"{name} {dtype} whole: worst relative error {worst:.2e}")
    assert all(eng.manager.free_pages(g) == eng.num_pages for g in range(len(eng.manager.groups)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_last_32_tokens_one_by_one(model_dirs, name, dtype):
    reqs = _requests(name)
    eng = _engine(model_dirs[name], dtype, max_tokens=208)
    got, routing = H.run_trace(eng, H.trace_tail_decode(reqs, 32))
    worst = H.compare_with_plain(model_dirs[name], reqs, got, routing, dtype)
    print(f"{name} {dtype} tail decode: worst relative error {worst:.2e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_portions_of_changing_size(model_dirs, name, dtype):
    reqs = _requests(name)
    eng = _engine(model_dirs[name], dtype, max_tokens=208)
    got, routing = H.run_trace(eng, H.trace_portions(reqs, random.Random(3)))
    worst = H.compare_with_plain(model_dirs[name], reqs, got, routing, dtype)
    print(f"{name} {dtype} portions: worst relative error {worst:.2e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_mixed_batches_reusing_pages(model_dirs, name, dtype):
    rng = random.Random(7)
    lengths = LENGTHS[name] + [rng.randrange(1, max(LENGTHS[name])) for _ in range(6)]
    reqs = H.random_requests(rng, VOCAB[name], lengths)
    # four live requests of the longest length fit, nothing more: every page is handed out many times
    longest = -(-max(lengths) // 16) * 16
    eng = _engine(model_dirs[name], dtype, max_tokens=4 * longest)
    steps = H.trace_mixed(reqs, rng, max_live=4)
    assert any(len(s["entries"]) >= 3 for s in steps)
    got, routing = H.run_trace(eng, steps)
    worst = H.compare_with_plain(model_dirs[name], reqs, got, routing, dtype)
    print(f"{name} {dtype} mixed: worst relative error {worst:.2e}")
    total_pages_needed = sum(-(-n // 16) for n in lengths)
    assert total_pages_needed > eng.num_pages, "the trace must need more pages than the pool has"


@pytest.mark.parametrize("name", NAMES)
def test_cutting_does_not_change_float32_logits(model_dirs, name):
    """In 32-bit every reduction has a fixed order per position, so whole, decoded and portioned runs
    agree far more closely than any of them agrees with another implementation."""
    reqs = _requests(name, seed=5)
    eng = _engine(model_dirs[name], "float32", max_tokens=208)
    whole, _ = H.run_trace(eng, H.trace_whole(reqs))
    cut, _ = H.run_trace(eng, H.trace_portions(reqs, random.Random(1)))
    worst = max(H.rel_err(cut[k], whole[k]) for k in whole)
    print(f"{name}: whole vs portions, float32: {worst:.2e}")
    assert worst < 2e-6


def test_a_checkpoint_stored_in_float32_served_in_bfloat16(tmp_path):
    """Tensors stored in 32-bit stay 32-bit in bfloat16 mode: activations and cache are bfloat16, the products
    run on the mixed-precision FMA kernel.  Same tolerance as any bfloat16 run."""
    import jax_llm_examples_b200 as J

    folder = H.make_model_dir(tmp_path / "m", "tiny_b", seed=3, dtype=torch.float32)
    model = J.load_model(folder, "bfloat16", "cuda")
    assert model.lm_head.dtype == torch.float32 and model.blocks[0].mixer.w_qkv.dtype == torch.float32
    eng = J.Engine(model, max_tokens=160, page_size=16, max_slots=4)
    assert eng.kv[0].dtype == torch.bfloat16
    rng = random.Random(5)
    reqs = H.random_requests(rng, 384, [90, 31])
    got, routing = H.run_trace(eng, H.trace_mixed(reqs, rng, max_live=2))
    H.compare_with_plain(folder, reqs, got, routing, "bfloat16")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_tied_embeddings(tmp_path, dtype):
    import jax_llm_examples_b200 as J

    folder = H.make_model_dir(tmp_path / "m", "tiny_a", seed=6, tie_word_embeddings=True)
    model = J.load_model(folder, dtype, "cuda")
    assert model.lm_head.data_ptr() == model.embedding.data_ptr()
    eng = J.Engine(model, max_tokens=128, page_size=16, max_slots=2)
    reqs = H.random_requests(random.Random(8), 256, [40, 9])
    got, routing = H.run_trace(eng, H.trace_tail_decode(reqs, 8))
    H.compare_with_plain(folder, reqs, got, routing, dtype)


@pytest.mark.parametrize("dtype, tol", [("float32", 1e-5), ("bfloat16", 4e-2)])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_renumbering_the_experts_changes_nothing(model_dirs, name, dtype, tol):
    """The same experts under other numbers (router rows and expert matrices permuted alike) are the same
    model: the sort by expert, the grouped products' tile lists and the combine must not care which number an
    expert has.  (Only the order in which a token's experts are added may change.)"""
    import jax_llm_examples_b200 as J
    from safetensors.torch import load_file

    folder = model_dirs[name]
    from jax_llm_examples_b200.config import load_config_json

    cfg_json = load_config_json(folder)
    tensors = load_file(str(folder / "model.safetensors"))
    E = cfg_json["num_local_experts"]
    perm = torch.tensor(random.Random(11).sample(range(E), E))
    assert not torch.equal(perm, torch.arange(E))
    renumbered = {}
    for key, t in tensors.items():
        if key.endswith("feed_forward.router.weight") or ".feed_forward.experts." in key:
            t = t[perm]
        renumbered[key] = t
    reqs = H.random_requests(random.Random(12), VOCAB[name], [70, 33])
    rows = []
    for ts in (tensors, renumbered):
        model = J.model_from_tensors(cfg_json, ts, dtype)
        eng = J.Engine(model, max_tokens=128, page_size=16, max_slots=2)
        got, _ = H.run_trace(eng, H.trace_portions(reqs, random.Random(13)))
        rows.append(got)
    assert rows[0].keys() == rows[1].keys() and len(rows[0]) > 0
    worst = max(H.rel_err(rows[1][k], rows[0][k]) for k in rows[0])
    assert worst < tol, f"{name} {dtype}: relative difference {worst:.2e} after renumbering the experts"


def test_random_model_on_the_device_and_the_written_folder(tmp_path):
    """``random_model(draw_on="cpu")`` is the model of the folder that ``write_random_model`` writes for the same
    seed; drawn on the device (the default) it is another model, as its docstring says."""
    import jax_llm_examples_b200 as J

    cfg = J.preset("tiny_b")
    folder = J.write_random_model(tmp_path / "m", cfg, seed=9, norm_noise=0.1)
    from_folder = J.load_model(folder, "bfloat16", "cuda")
    same = J.random_model(cfg, 9, "bfloat16", "cuda", norm_noise=0.1, draw_on="cpu")
    other = J.random_model(cfg, 9, "bfloat16", "cuda", norm_noise=0.1)
    assert torch.equal(same.embedding, from_folder.embedding) and torch.equal(same.lm_head, from_folder.lm_head)
    assert torch.equal(same.blocks[3].mixer.w_qkv, from_folder.blocks[3].mixer.w_qkv)
    assert torch.equal(same.blocks[1].feed_forward.we_down, from_folder.blocks[1].feed_forward.we_down)
    assert not torch.equal(other.embedding, from_folder.embedding)
    with pytest.raises(ValueError, match="draw_on"):
        J.random_model(cfg, 9, draw_on="gpu")
