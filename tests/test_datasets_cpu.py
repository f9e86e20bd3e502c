"""Dataset files from captures and from the synthetic generators."""
import numpy as np
import torch

from ccbench_b200 import datasets as D


def test_sizes_and_labels():
    assert D.parse_size("512mb") == 512 << 20 and D.parse_size("4GB") == 4 << 30 and D.parse_size("100") == 100
    assert D.size_label(512 << 20) == "512mb" and D.size_label(4 << 30) == "4gb"


def test_captures_are_grouped_tiled_and_named(tmp_path):
    src = tmp_path / "rank_0"
    src.mkdir()
    torch.save(torch.arange(10, dtype=torch.bfloat16), src / "SP_ReduceScatter_fwd_activation_global_before.pt")
    torch.save({"t": torch.full((5,), 7.0)}, src / "PP_Comm_send_fwd_activation.pt")
    for i in range(3):
        torch.save(torch.full((4,), float(i)), src / f"DP_ReduceScatter_grad_shard_{i}.pt")
    np.arange(6, dtype=np.float32).tofile(src / "DP_AllGather_Input_weight_shard_0.bin")
    made = D.from_captures(src, tmp_path / "dataset", 256, verbose=False)
    assert set(made) == {"activation", "weight", "dp_grad"}
    act = np.fromfile(made["activation"], dtype=np.float32)
    assert made["activation"].name == "act_cache_256b.f32" and act.size == 64
    assert np.array_equal(act[:15], np.concatenate([np.arange(10), np.full(5, 7.0)]).astype(np.float32))
    assert np.array_equal(act[15:25], np.arange(10, dtype=np.float32))  # tiled
    g = np.fromfile(made["dp_grad"], dtype=np.float32)
    assert np.array_equal(g[:12], np.repeat(np.arange(3, dtype=np.float32), 4))


def test_synthetic_and_rank_split(tmp_path):
    made = D.synthetic(tmp_path / "dataset", 1 << 16, verbose=False)
    assert set(made) == set(D.CATEGORIES)
    for p in made.values():
        assert p.stat().st_size == 1 << 16
    again = D.synthetic(tmp_path / "again", 1 << 16, verbose=False)
    assert np.array_equal(np.fromfile(made["dp_grad"], np.float32), np.fromfile(again["dp_grad"], np.float32))
    parts = D.per_rank_folder(made["dp_grad"], tmp_path / "ranks", 3, 1 << 15)
    data = np.fromfile(made["dp_grad"], np.float32)
    r1 = np.fromfile(parts[1], np.float32)
    assert r1.size == (1 << 15) // 4 and np.array_equal(r1, data[r1.size:2 * r1.size])
    r2 = np.fromfile(parts[2], np.float32)
    assert np.array_equal(r2, data[(np.arange(r2.size) + 2 * r2.size) % data.size])
