"""The grouping of device-timeline records into launches and their summary over several steps (no GPU: records are
made by hand in the layout that the kernels write)."""

import numpy as np
import pytest


def _record(kernel_id, grid, first, start, waited, end, marks=(0, 0, 0, 0)):
    what = kernel_id | (grid[0] << 8) | (grid[1] << 24) | (grid[2] << 40)
    if first:
        what -= 1 << 63  # the top bit, in a signed 64-bit word
    return [what, start, waited, end, *marks]


class _Timeline:
    """DeviceTimeline without a device: ``records()`` returns what the test gives it."""

    def __init__(self, rows):
        self.rows = np.array(rows, dtype=np.int64)

    def records(self):
        return self.rows


@pytest.fixture
def timeline_class():
    from jax_llm_examples_b200.tracing import DeviceTimeline

    class Fake(_Timeline, DeviceTimeline):
        pass

    return Fake


def test_records_of_one_grid_form_one_launch_however_they_interleave(timeline_class):
    # kernel 2 (add_rmsnorm, 1 block) then kernel 4 (gemm_stream, 2 x 1 x 2 = 4 blocks) whose blocks start early, while
    # the norm still runs, and a second launch of the same product later
    rows = [
        _record(2, (1, 1, 1), True, 1000, 1500, 9000, (1600, 0, 0, 0)),
        _record(4, (2, 1, 2), True, 2000, 9500, 20000),
        _record(4, (2, 1, 2), False, 2100, 9600, 21000),
        _record(4, (2, 1, 2), False, 2200, 9550, 19000),
        _record(4, (2, 1, 2), False, 8000, 9700, 22000),
        _record(4, (2, 1, 2), True, 30000, 30100, 40000),
        _record(4, (2, 1, 2), False, 30010, 30200, 41000),
        _record(4, (2, 1, 2), False, 30020, 30150, 39000),
        _record(4, (2, 1, 2), False, 30030, 30120, 42000),
    ]
    launches = timeline_class(rows).launches()
    assert [(g["kernel"], g["grid"], g["blocks"], g["occurrence"]) for g in launches] == [
        ("add_rmsnorm", (1, 1, 1), 1, 0), ("gemm_stream", (2, 1, 2), 4, 0), ("gemm_stream", (2, 1, 2), 4, 1)]
    norm, first, second = launches
    assert norm["start"] == 0.0 and norm["ready"] == 0.5 and norm["end"] == 8.0 and norm["marks"] == [0.6, None, None, None]
    assert first["start"] == 1.0 and first["ready"] == 8.5 and first["end"] == 21.0 and first["marks"] is None
    assert second["ready"] == 29.1 and second["end"] == 41.0


def test_summary_takes_medians_per_launch_and_what_each_adds(timeline_class):
    def step(shift, norm_end, gemm_end):
        rows = [
            _record(2, (1, 1, 1), True, shift + 1000, shift + 2000, shift + norm_end, (shift + 2500, 0, 0, 0)),
            _record(4, (1, 1, 1), True, shift + 1500, shift + norm_end + 500, shift + gemm_end),
        ]
        return timeline_class(rows).launches()

    rows = timeline_class.summary([step(0, 9000, 20000), step(7, 10000, 23000), step(99, 11000, 22000)])
    assert [r["kernel"] for r in rows] == ["add_rmsnorm", "gemm_stream"]
    norm, gemm = rows
    assert norm["busy"] == 8.0 and norm["early"] == 1.0 and norm["marks"][0] == 0.5
    assert gemm["busy"] == pytest.approx(10.5) and gemm["adds"] == pytest.approx(11.0) and gemm["early"] == pytest.approx(9.0)
    assert "add_rmsnorm" in timeline_class.table(rows)
