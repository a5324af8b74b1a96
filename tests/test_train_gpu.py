"""End-to-end training steps on the GPU: bf16 kernels vs the fp32 CPU path of the same graph,
CUDA-graph replay, dropout determinism in backward."""
import pytest
import torch

from tnn_b200.models import zoo
from tnn_b200.nn.loss import CrossEntropyLoss
from tnn_b200.ops import _lib
from tnn_b200.trainer import Trainer
from tnn_b200.utils.config import TrainingConfig

pytestmark = pytest.mark.gpu


def tiny(drop):
    return zoo.gpt2(128, 2, 2, "t", seq_len=128, vocab=203, drop=drop)


def test_gpt_step_matches_cpu_reference():
    torch.manual_seed(0)
    ids = torch.randint(0, 203, (2, 128))
    labels = torch.randint(0, 203, (2, 128))
    gc = tiny(0.0).compile(device="cpu", seed=7)
    gg = tiny(0.0).compile(device="cuda", seed=7)
    assert torch.equal(gc.master_flat, gg.master_flat.cpu())
    # the CPU copy must see bf16-rounded weights, like the kernels do
    gc.params_flat.copy_(gg.params_flat.float().cpu())
    out_c = gc.forward({"input": ids})["output"]
    out_g = gg.forward({"input": ids.cuda()})["output"]
    _lib.check_status()
    assert (out_g.float().cpu() - out_c).abs().max() < 0.15 * out_c.abs().max()
    lc, grad_c = CrossEntropyLoss().compute(out_c, labels)
    lg, grad_g = CrossEntropyLoss().compute(out_g, labels.cuda())
    assert abs(float(lc) - float(lg)) < 0.05
    gc.backward({"output": grad_c})
    gg.backward({"output": grad_g})
    _lib.check_status()
    a, b = gc.grads_flat, gg.grads_flat.cpu()
    cos = torch.nn.functional.cosine_similarity(a, b, dim=0)
    assert cos > 0.99, float(cos)
    rel = (a - b).norm() / a.norm()
    assert rel < 0.1, float(rel)


def test_loss_decreases_with_dropout_and_graph_replay():
    torch.manual_seed(1)
    g = tiny(0.1).compile(device="cuda", seed=3)
    cfg = TrainingConfig.from_dict({"model_name": "t", "batch_size": 4, "optimizer": {"type": "adamw", "learning_rate": 2e-3}})
    t = Trainer(cfg, graph=g, log=False)
    seq = torch.randint(0, 203, (4, 129))
    d, l = seq[:, :-1].contiguous(), seq[:, 1:].contiguous()
    l0 = float(t.train_step(d, l).item())
    t.enable_cuda_graph(d, l)
    assert t.launches_per_step > 20
    for _ in range(30):
        loss = t.train_step(d, l)
    l1 = float(loss.item())
    _lib.check_status()
    assert l1 < l0 - 0.5, (l0, l1)
    t.close()


def test_vocab_head_uses_padded_logits():
    g = tiny(0.0).compile(device="cuda", seed=2)
    out = g.forward({"input": torch.randint(0, 203, (1, 128)).cuda()})["output"]
    assert out.shape == (1, 128, 203) and out.stride(1) % 64 == 0


@pytest.mark.parametrize("graphed", [False, True])
def test_overlapped_update_equals_update_after_backward(graphed, monkeypatch):
    """The optimizer buckets launched on a second stream during backward (nn/optim.py OverlappedUpdate) leave the
    same weights as one update after backward, eagerly and under CUDA-graph replay."""
    from tnn_b200.nn.optim import OverlappedUpdate

    def run(overlap):
        monkeypatch.setenv("TNNB_OVERLAP_UPDATE", "1" if overlap else "0")
        monkeypatch.setenv("TNNB_UPDATE_MIN_BUCKET", "1024")
        torch.manual_seed(5)
        g = tiny(0.0).compile(device="cuda", seed=3)
        cfg = TrainingConfig.from_dict({"model_name": "t", "batch_size": 4,
                                        "optimizer": {"type": "adamw", "learning_rate": 1e-3, "weight_decay": 0.1}})
        t = Trainer(cfg, graph=g, log=False)
        assert isinstance(t.optimizer, OverlappedUpdate) == overlap
        if overlap:
            assert len(t.optimizer.spans) > 1
        seq = torch.randint(0, 203, (4, 129))
        d, l = seq[:, :-1].contiguous(), seq[:, 1:].contiguous()
        t.train_step(d, l)
        if graphed:
            t.enable_cuda_graph(d, l)
        for _ in range(6):
            loss = t.train_step(d, l)
        torch.cuda.synchronize()
        _lib.check_status()
        assert float(g.grads_flat.abs().max()) == 0.0  # cleared, whoever did it
        out = g.master_flat.clone(), float(loss.item()), t.optimizer.step_count
        t.close()
        return out

    (wa, la, na), (wb, lb, nb) = run(True), run(False)
    assert na == nb
    assert abs(la - lb) < 2e-2
    assert float((wa - wb).norm() / wb.norm()) < 2e-3


@pytest.mark.parametrize("graphed", [False, True])
def test_prefetched_batches_give_the_same_training(graphed):
    """Trainer.prefetch uploads the next batch on a copy stream while the current step runs; the losses must be
    those of plain train_step calls on the same batches, eagerly and under CUDA-graph replay."""
    def run(prefetch):
        torch.manual_seed(11)
        g = tiny(0.0).compile(device="cuda", seed=3)
        cfg = TrainingConfig.from_dict({"model_name": "t", "batch_size": 4, "optimizer": {"type": "adamw", "learning_rate": 1e-3}})
        t = Trainer(cfg, graph=g, log=False)
        gen = torch.Generator().manual_seed(2)
        batches = []
        for _ in range(8):
            seq = torch.randint(0, 203, (4, 129), generator=gen)
            batches.append((seq[:, :-1].contiguous().pin_memory(), seq[:, 1:].contiguous().pin_memory()))
        if graphed:
            t.enable_cuda_graph(*batches[0])
        losses = []
        for i, (d, l) in enumerate(batches):
            loss = t.train_step(d, l)
            if prefetch and i + 1 < len(batches):
                t.prefetch(*batches[i + 1])
            losses.append(float(loss.item()))
        _lib.check_status()
        t.close()
        return losses

    a, b = run(True), run(False)
    assert len(a) == 8 and max(abs(x - y) for x, y in zip(a, b)) < 2e-2, (a, b)
    assert abs(a[0] - a[-1]) > 1e-3  # different batches and updates: the losses move


def test_allocation_tracker_reports_peak_per_edge():
    """The allocation hook brackets every edge's forward and backward pass with allocator readings: a training
    forward keeps memory (what it saved), its backward gives it back, and every peak is at least what was kept."""
    import torch
    from tnn_b200.models import zoo
    g = zoo.gpt2(128, 2, 2, "t", seq_len=128, vocab=203, drop=0.0).compile(device="cuda", seed=0)
    g.set_training(True)
    trk = g.track_memory(True)
    ids = torch.randint(0, 203, (4, 128), device="cuda")
    out = g.forward({"input": ids})["output"]
    g.backward({"output": torch.randn_like(out)})
    rows = trk.peak_per_edge()
    assert len(rows) == len(g.segments)
    kept = sum(d["forward_kept"] for d in rows.values())
    freed = sum(d["backward_freed"] for d in rows.values())
    assert kept > 4 * 128 * 128 * 2 * 4 and freed > 0
    assert all(d["forward_peak"] >= d["forward_kept"] for d in rows.values())
    assert "fwd peak MiB" in trk.format()
    g.track_memory(False)
    assert g.alloc_hook is None
