"""Vision tower oracle: patch ordering, resize rule, rotary table, merge-group layout (CPU)."""
import torch

from cuteafd_b200.ref.vision import (VisionSpec, init_vision_weights, patch_order, position_rows, rgb_to_patches, rope_table, smart_grid,
                                     vision_forward)


def test_patch_order_walks_merge_groups():
    ys, xs = patch_order(4, 6, 2)
    assert list(zip(ys[:8].tolist(), xs[:8].tolist())) == [(0, 0), (0, 1), (1, 0), (1, 1), (0, 2), (0, 3), (1, 2), (1, 3)]
    assert sorted(zip(ys.tolist(), xs.tolist())) == [(y, x) for y in range(4) for x in range(6)]


def test_rgb_patches_follow_the_order_and_the_lut():
    spec = VisionSpec(patch=4, merge=2, image_mean=(0.5, 0.4, 0.3), image_std=(0.2, 0.25, 0.5))
    g = torch.Generator().manual_seed(0)
    rgb = torch.randint(0, 256, (8, 16, 3), generator=g, dtype=torch.uint8)
    p = rgb_to_patches(rgb, spec)
    assert p.shape == (2 * 4, 48)
    ys, xs = patch_order(2, 4, 2)
    for row in (0, 3, 5):
        y0, x0 = int(ys[row]) * 4, int(xs[row]) * 4
        for c, py, px in ((0, 0, 0), (1, 2, 3), (2, 3, 1)):
            want = (float(rgb[y0 + py, x0 + px, c]) / 255 - spec.image_mean[c]) / spec.image_std[c]
            assert abs(float(p[row, c * 16 + py * 4 + px]) - want) < 1e-6


def test_smart_grid_keeps_whole_merge_groups_and_token_bounds():
    spec = VisionSpec(patch=16, merge=2, min_tokens=4, max_tokens=64)
    for h, w in ((10, 10), (640, 480), (4000, 300), (37, 1999)):
        gh, gw = smart_grid(h, w, spec)
        assert gh % 2 == 0 and gw % 2 == 0
        assert 4 <= gh * gw // 4 <= 64 or gh * gw // 4 <= 64 + max(gh, gw)       # rounding may overshoot by less than a row of groups
    assert smart_grid(640, 480, VisionSpec(patch=16, merge=2, max_tokens=4096)) == (40, 30)


def test_rope_table_splits_rows_and_columns():
    spec = VisionSpec(head_dim=16, merge=2)
    cs = rope_table(2, 4, spec)
    ys, xs = patch_order(2, 4, 2)
    assert cs.shape == (8, 16)
    # angle 0 of the row half follows y, angle 0 of the column half follows x (inverse frequency 1)
    assert torch.allclose(cs[:, 0], ys.float().cos()) and torch.allclose(cs[:, 8], ys.float().sin())
    assert torch.allclose(cs[:, 4], xs.float().cos()) and torch.allclose(cs[:, 12], xs.float().sin())


def test_position_table_resample_is_identity_on_its_own_grid():
    spec = VisionSpec(hidden=8, pos_grid=4, merge=2)
    t = torch.randn(16, 8)
    r = position_rows(t, 4, 4, spec)
    ys, xs = patch_order(4, 4, 2)
    assert torch.allclose(r, t.reshape(4, 4, 8)[ys, xs], atol=1e-6)


def test_forward_is_invariant_to_which_image_shares_the_batch_and_depends_on_all_patches():
    for kw in (dict(), dict(norm="rmsnorm", mlp="swiglu", qk_norm=True, pos_grid=3)):
        spec = VisionSpec(hidden=32, depth=2, n_heads=2, head_dim=16, intermediate=48, patch=4, out_hidden=24, **kw)
        w = init_vision_weights(spec, 1)
        g = torch.Generator().manual_seed(2)
        rgb = torch.randint(0, 256, (16, 8, 3), generator=g, dtype=torch.uint8)
        p = rgb_to_patches(rgb, spec)
        out = vision_forward(spec, w, p, 4, 2)
        assert out.shape == (2, 24) and torch.isfinite(out).all()
        p2 = p.clone()
        p2[-1] += 1.0                                     # the last patch belongs to the second merge group
        out2 = vision_forward(spec, w, p2, 4, 2)
        assert (out2[0] - out[0]).abs().max() > 1e-6      # bidirectional: the first group's row sees it too
