"""Host-side decisions of the routed feed-forward (no GPU): where a step's shared expert runs, and what a norm that
routes for the part is offered."""

import types

import torch


def _experts(shared_like_experts: bool):
    from jax_llm_examples_b200.parts import DenseSwiGLU, RoutedExperts

    E, D, F = 4, 32, 16
    g = torch.Generator().manual_seed(0)
    w = lambda *shape: torch.randn(*shape, generator=g).to(torch.bfloat16)  # noqa: E731
    shared = DenseSwiGLU(w(2 * F, D), w(D, F)) if shared_like_experts else DenseSwiGLU(w(2 * 24, D), w(D, 24))
    return RoutedExperts(torch.randn(E, D, generator=g), w(E, 2 * F, D), w(E, D, F), top_k=2, shared=shared)


def _ctx(workspace):
    return types.SimpleNamespace(workspace=workspace)


def test_where_the_shared_expert_runs():
    import importlib

    linear = importlib.import_module("jax_llm_examples_b200.parts.linear")

    ffn, ws = _experts(True), object()
    assert ffn.merged
    # one row: a group of the routed experts' products; a few rows up to the streaming limit: a second stream
    assert ffn.FORK_MIN_ROWS == 2 and ffn.placement(_ctx(ws), 1) == (False, True)
    assert ffn.placement(_ctx(ws), ffn.FORK_MIN_ROWS) == (True, False) and ffn.placement(_ctx(ws), linear.STREAM_MAX_ROWS) == (True, False)
    # between the streaming limit and a prompt portion worth overlapping: one after the other; then beside again
    assert ffn.placement(_ctx(ws), linear.STREAM_MAX_ROWS + 1) == (False, False)
    assert ffn.placement(_ctx(ws), ffn.OVERLAP_MIN_ROWS) == (True, False)
    # no workspace (so no second stream): never beside, a group while the step is small
    assert ffn.placement(_ctx(None), 8) == (False, True) and ffn.placement(_ctx(None), 4096) == (False, False)
    # a shared expert of another shape cannot ride as a group
    other = _experts(False)
    assert not other.merged and other.placement(_ctx(ws), 1) == (False, False) and other.placement(_ctx(ws), 8) == (True, False)


def test_the_router_request_offers_the_sort_and_gather_and_needs_a_workspace_for_it():
    ffn = _experts(True)
    w_router, k, offer = ffn.router_request()
    assert w_router is ffn.w_router and k == 2 and callable(offer)
    assert offer(_ctx(None), 1) is None  # the ticket counter lives in the workspace
