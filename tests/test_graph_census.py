"""Graph-bank census: row buckets, capture watch after sealing, timing arms (CPU only)."""
from cuteafd_b200.utils.graph_census import GraphCensus, bucket_rows


def test_row_buckets():
    assert [bucket_rows(n) for n in (1, 2, 4, 5, 16, 17, 64, 65, 128, 129)] == [1, 4, 4, 16, 16, 64, 64, 128, 128, 192]


def test_census_counts_and_reports_steady_state_captures():
    c = GraphCensus()
    for key in ("a", "b"):
        c.captured(key, launches=12)
        for _ in range(3):
            c.replayed(key)
    c.ran_eager("a")
    c.seal()
    c.replayed("a")
    assert c.snapshot()["steady_state_captures"] == 0
    c.captured("c")                                    # a shape nobody warmed: reported
    s = c.snapshot()
    assert s["steady_state_captures"] == 1 and s["shapes"] == 3 and s["captures"] == 3 and s["replays"] == 7 and s["eager_runs"] == 1
    c.arms("a", eager_ms=2.0, graph_ms=1.5)
    assert c.snapshot()["arms"]["a"]["launch_bound_share"] == 0.25 and c.snapshot()["arms"]["a"]["launches"] == 12
    c.invalidate()
    assert not c.sealed and c.snapshot()["shapes"] == 0
