"""The C++ host runtime: wire format (golden bytes built independently with ``struct``), typed config, profiler merge,
allocators, data loaders on synthetic files, tokenizer, partitioner, CPU oracle engine against torch autograd, and
the schedulers' arithmetic."""
import json
import math
import os
import struct

import numpy as np
import pytest
import torch

from tnn_b200.host import H


# ------------------------------------------------------------------------------------ wire format
def _golden_job_message(cmd, pid, uid, dtype, dims, raw):
    b = struct.pack("<HI", cmd, 1)                                  # u16 command, u32 payload index (1 = Job)
    b += struct.pack("<QQ", pid, 1)                                 # pid, tensor count
    b += struct.pack("<Q", len(uid)) + uid.encode()                 # string = u64 length + bytes
    b += struct.pack("<IQ", dtype, len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + raw
    return b


def test_message_bytes_match_the_documented_layout():
    cmd = H.command_code("FORWARD_JOB")
    raw = np.arange(6, dtype=np.float32).tobytes()
    msg = {"command": cmd, "kind": 1, "job": {"pid": 3, "tensors": [("x", (H.dtype_code("FP32"), [2, 3], raw))]}}
    wire = H.serialize_message(msg)
    assert wire == _golden_job_message(cmd, 3, "x", H.dtype_code("FP32"), [2, 3], raw)
    back = H.parse_message(wire)
    assert back["command_name"] == "FORWARD_JOB" and back["job"]["pid"] == 3
    name, (dt, shape, data) = back["job"]["tensors"][0]
    assert (name, dt, list(shape), data) == ("x", H.dtype_code("FP32"), [2, 3], raw)
    # string, bool and stage-config payloads round-trip
    for m in ({"command": H.command_code("SAVE_TO_FILE"), "kind": 2, "text": "model_snapshots/stage0"},
              {"command": H.command_code("CONFIG_RECEIVED"), "kind": 3, "flag": True},
              {"command": H.command_code("CONFIG_TRANSFER"), "kind": 5,
               "stage": {"graph_state": b"TNNG....", "input_uids": ["input"], "output_uids": ["h3"], "optimizer_config": "{}",
                         "scheduler_config": "{}", "next_stage": "{}", "prev_stage": "{}", "coordinator": "{}"}}):
        out = H.parse_message(H.serialize_message(m))
        for k, v in m.items():
            if k == "stage":
                assert out["stage"]["input_uids"] == ["input"] and bytes(out["stage"]["graph_state"]) == b"TNNG...."
            else:
                assert out[k] == v


def test_packets_have_36_byte_headers_and_reassemble_out_of_order():
    assert H.PACKET_HEADER_SIZE == 36
    payload = bytes(range(256)) * 9
    wire = H.serialize_message({"command": H.command_code("SAVE_TO_FILE"), "kind": 2, "text": payload.decode("latin1")})
    packets = H.slice_message(wire, 42, 500)
    assert len(packets) == math.ceil(len(wire) / 500)
    h0 = H.parse_packet_header(packets[0])
    assert h0["msg_serial_id"] == 42 and h0["msg_length"] == len(wire) and h0["total_packets"] == len(packets)
    assert len(packets[0]) == 36 + 500
    # golden header of packet 1: u8 ver, u8 type, u8 endian, u64 packet_len, u64 msg_len, u64 id, u32 offset, u32 total, u8 compression
    assert packets[1][:36] == struct.pack("<BBBQQQIIB", 1, 0, 1, 500, len(wire), 42, 1, len(packets), 0)
    agg = H.Aggregator()
    done = None
    for p in reversed(packets):
        r = agg.feed(p)
        if r is not None:
            done = r
    assert done is not None and done[0] == 42 and bytes(done[1]) == wire and agg.pending() == 0


def _packet(packet_len, msg_len, msg_id, offset, total, payload):
    return struct.pack("<BBBQQQIIB", 1, 0, 1, packet_len, msg_len, msg_id, offset, total, 0) + payload


def test_aggregator_rejects_malformed_headers():
    """Header fields arrive from the network: a fragment longer than its message, an offset that wraps, a message
    or packet count beyond the receiver's limits must all be refused before anything is allocated or copied."""
    import pytest
    bad = [
        _packet(4096, 8, 1, 1, 2, b"x" * 4096),                 # last fragment longer than the message (used to underflow)
        _packet(8, 8, 2, 5, 2, b"x" * 8),                        # packet index >= packet count
        _packet(8, 16, 3, 0, 0, b"x" * 8),                       # zero packets
        _packet(4, 8, 4, 2, 4, b"x" * 4),                        # fragment 2 of 4 x 4 bytes lies beyond an 8-byte message
        _packet(1, 1 << 40, 5, 0, 1 << 20, b"x"),                # announces a terabyte
        _packet(1, 64, 6, 0, 100, b"x"),                         # more packets than bytes
        _packet(2**63, 2**63 + 8, 7, 3, 4, b""),                 # offset arithmetic would wrap
    ]
    for pkt in bad:
        agg = H.Aggregator(1 << 20, 1 << 10)
        with pytest.raises(Exception):
            agg.feed(pkt)
    # limits are per receiver: the same well-formed message passes a roomy aggregator and is refused by a tight one
    wire = bytes(300)
    pk = H.slice_message(wire, 9, 100)
    tight = H.Aggregator(256, 16)
    with pytest.raises(Exception):
        tight.feed(pk[0])
    roomy = H.Aggregator(1 << 20, 16)
    out = [roomy.feed(p) for p in pk]
    assert out[-1] is not None and bytes(out[-1][1]) == wire


def test_tconfig_type_tags_round_trip_and_profiler_merge():
    c = H.TConfig()
    c.name, c.type = "fc", "dense"
    c.set("input_features", "unsigned long", 784)
    c.set("use_bias", "bool", True)
    c.set("activation", "string", "relu")
    text = c.dump()
    d = json.loads(text)
    assert d["parameters"]["input_features"] == {"type": "unsigned long", "value": 784} and d["type"] == "dense"
    assert H.tconfig_normalize(text) == text and H.TConfig.parse(text).get("activation") == "relu"
    a, b = H.Profiler(), H.Profiler()
    a.set_start_time(1_000_000)
    b.set_start_time(3_000_000)      # rank b started 2 ms later
    a.add_event(1, 1_500_000, 2_500_000, "send", "r0")
    b.add_event(1, 3_200_000, 3_900_000, "recv", "r1")
    a.merge(b)
    a.sort()
    ev = a.events()
    assert len(ev) == 2 and ev[0][3] == "recv" and ev[0][0] == 1_200_000   # shifted by the start-time difference
    assert "Type: COMMUNICATION" in a.log_lines()[0] and "Duration: 0.700 ms" in a.log_lines()[0]


# ------------------------------------------------------------------------------------ allocators
def test_pool_allocator_reuses_buckets_and_arena_flips_sides():
    pool = H.PoolAllocator(1 << 16, 256)
    a, b = pool.allocate(1000), pool.allocate(3000)
    assert a == 0 and b == 1024 and pool.used() == 1024 + 3072
    pool.release(a)
    assert pool.allocate(900) == 0 and pool.peak() == 4096
    assert pool.allocate(1 << 20) < 0                                   # exhausted: negative offset, no exception
    arena = H.DoubleEndedArena(1 << 16, 256)
    x = arena.allocate(4096)
    arena.flip()
    y = arena.allocate(4096)
    assert x == 0 and y == (1 << 16) - 4096 and arena.side() == 1
    arena.release(x)
    arena.release(y)
    assert arena.used() == 0 and arena.free_blocks() == 1


# ------------------------------------------------------------------------------------ data loaders
def test_cifar_mnist_and_token_loaders_on_synthetic_files(tmp_path):
    rng = np.random.default_rng(0)
    # CIFAR-10: records of 1 label byte + 3072 bytes CHW u8 -> NHWC float / 255
    recs = []
    for i in range(10):
        img = rng.integers(0, 256, (3, 32, 32), dtype=np.uint8)
        recs.append((i % 10, img))
    f = tmp_path / "data_batch_1.bin"
    f.write_bytes(b"".join(bytes([l]) + im.tobytes() for l, im in recs))
    ld = H.Loader.cifar10([str(f)], 4, False, 0, 2)
    assert len(ld) == 10 and list(ld.sample_shape()) == [32, 32, 3]
    x, y = ld.next()
    assert x.shape == (4, 32, 32, 3) and y.tolist() == [0, 1, 2, 3]
    assert np.allclose(x[1], recs[1][1].transpose(1, 2, 0).astype(np.float32) / 255.0)
    # CIFAR-100: coarse, fine, pixels; fine labels by default
    f100 = tmp_path / "train.bin"
    f100.write_bytes(b"".join(bytes([7, 50 + i]) + recs[i][1].tobytes() for i in range(4)))
    _, y100 = H.Loader.cifar100([str(f100)], False, 4, False, 0, 0).next()
    assert y100.tolist() == [50, 51, 52, 53]
    # MNIST csv with a header line
    rows = ["label," + ",".join(f"p{i}" for i in range(784))]
    for i in range(5):
        rows.append(str(i) + "," + ",".join(str((i * 7 + j) % 256) for j in range(784)))
    csv = tmp_path / "train.csv"
    csv.write_text("\n".join(rows) + "\n")
    xm, ym = H.Loader.mnist_csv(str(csv), 5, False, 0, 0).next()
    assert xm.shape == (5, 28, 28, 1) and ym.tolist() == [0, 1, 2, 3, 4] and abs(xm[1, 0, 1, 0] - 8 / 255) < 1e-6
    # token stream: random windows, labels shifted by one
    toks = np.arange(5000, dtype=np.uint16)
    tb = tmp_path / "tokens.bin"
    toks.tofile(tb)
    xt, yt = H.Loader.tokens(str(tb), 64, 3, 1, 2).next()
    assert xt.shape == (3, 64) and yt.shape == (3, 64)
    assert np.array_equal(yt[:, :-1], xt[:, 1:].astype(np.int32)) and np.array_equal(yt[:, 0], xt[:, 0].astype(np.int32) + 1)


def test_tokenizer_vocab_file(tmp_path):
    from tnn_b200.data.tokenizer import Tokenizer, write_vocab

    path = str(tmp_path / "vocab.bin")
    write_vocab(path, [b"Hello", b",", b" world", b"!"])
    raw = open(path, "rb").read()
    assert raw[:4] == struct.pack("<I", 4) and raw[4:8] == struct.pack("<I", 5) and raw[8:13] == b"Hello"
    tok = Tokenizer(path)
    assert len(tok) == 4 and tok.decode([0, 1, 2, 3]) == "Hello, world!"
    assert H.Tokenizer(path).decode([2, 3]) == b" world!"  # the C++ class returns raw bytes (tokens need not be valid UTF-8)


# ------------------------------------------------------------------------------------ partitioner
def test_partition_largest_remainder_and_empty_partition_error():
    ir = {"nodes": [f"n{i}" for i in range(8)], "inputs": [0], "outputs": [7],
          "edges": [(i, [i], [i + 1]) for i in reversed(range(7))]}            # edges listed back to front
    order = H.topo_sort(ir)
    assert list(order["edge_perm"]) == [6, 5, 4, 3, 2, 1, 0]                    # Kahn order restores the chain
    assert H.resolve_layer_counts([1.0, 1.0], 7) == [4, 3]                      # 3.5 / 3.5: the remainder goes to the lower index
    assert H.resolve_layer_counts([1.0, 2.0, 1.0], 7) == [2, 3, 2]              # 1.75 / 3.5 / 1.75
    with pytest.raises(RuntimeError):                                           # a ratio that rounds to zero layers is an error
        H.resolve_layer_counts([0.01, 0.01, 10.0], 7)
    parts = H.partition(ir, [1.0, 2.0])
    assert len(parts) == 2
    assert len(parts[0]["edges"]) + len(parts[1]["edges"]) == 7


# ------------------------------------------------------------------------------------ CPU oracle engine
def test_cpu_engine_conv_bn_pool_match_torch_autograd():
    torch.manual_seed(0)
    x = torch.randn(2, 9, 8, 5, requires_grad=True)          # NHWC
    w = torch.randn(6, 3, 3, 5, requires_grad=True)          # O, KH, KW, I
    b = torch.randn(6, requires_grad=True)
    y = torch.from_numpy(H.cpu.conv2d_fwd(x.detach().numpy(), w.detach().numpy(), b.detach().numpy(), 2, 1, 1, 0))
    ref = torch.nn.functional.conv2d(x.permute(0, 3, 1, 2), w.permute(0, 3, 1, 2), b, stride=(2, 1), padding=(1, 0)).permute(0, 2, 3, 1)
    assert torch.allclose(y, ref, atol=1e-4)
    dy = torch.randn_like(ref)
    ref.backward(dy)
    dx = torch.from_numpy(H.cpu.conv2d_dgrad(dy.numpy(), w.detach().numpy(), list(x.shape), 2, 1, 1, 0))
    assert torch.allclose(dx, x.grad, atol=1e-4)
    dw, db = np.zeros(w.shape, np.float32), np.zeros(6, np.float32)
    H.cpu.conv2d_wgrad(x.detach().numpy(), dy.numpy(), dw, db, 2, 1, 1, 0)
    assert torch.allclose(torch.from_numpy(dw), w.grad, atol=1e-3) and torch.allclose(torch.from_numpy(db), b.grad, atol=1e-4)
    # max pool: window clipped to the image, mask = window-relative index
    xp = torch.randn(1, 5, 5, 2)
    yp, idx = H.cpu.pool2d_fwd(xp.numpy(), True, 3, 3, 2, 2, 1, 1)
    refp = torch.nn.functional.max_pool2d(xp.permute(0, 3, 1, 2), 3, 2, 1).permute(0, 2, 3, 1)
    assert torch.allclose(torch.from_numpy(yp), refp) and idx.min() >= 0 and idx.max() < 9
    # softmax cross-entropy
    z = torch.randn(7, 11, requires_grad=True)
    lab = torch.randint(0, 11, (7,))
    loss, grad, corrects = H.cpu.softmax_ce(z.detach().numpy(), lab.numpy().astype(np.int32))
    assert corrects == int((z.argmax(1) == lab).sum())
    ref_loss = torch.nn.functional.cross_entropy(z, lab)
    ref_loss.backward()
    assert abs(float(loss) - float(ref_loss.detach())) < 1e-5 and torch.allclose(torch.from_numpy(grad), z.grad, atol=1e-6)


# ------------------------------------------------------------------------------------ schedulers
class _Opt:
    def __init__(self, lr):
        self.learning_rate = lr

    def get_learning_rate(self):
        return self.learning_rate

    def set_learning_rate(self, lr):
        self.learning_rate = lr


def test_scheduler_arithmetic_including_the_unsigned_wrap():
    from tnn_b200.nn import schedulers as S

    o = _Opt(1.0)
    s = S.StepLR(o, step_size=2, gamma=0.5)
    lrs = []
    for _ in range(5):
        s.step()
        lrs.append(o.learning_rate)
    assert lrs == [1.0, 0.5, 0.5, 0.25, 0.25]                   # multiplies the CURRENT rate every step_size steps
    o = _Opt(1.0)
    s = S.CosineAnnealingLR(o, T_max=4, eta_min=0.0)
    vals = []
    for _ in range(5):
        s.step()
        vals.append(round(o.learning_rate, 6))
    assert vals[3] == 1.0 and vals[1] == 0.5                     # uses step % T_max: the rate jumps back at T_max
    o = _Opt(0.8)
    s = S.LinearWarmup(o, warmup_steps=4, start_lr=0.0)
    assert abs(o.learning_rate - 0.2) < 1e-6                     # base / warmup at construction (float32 arithmetic, as in the reference)
    s.step()
    assert abs(o.learning_rate - 0.8 * 2 / 4) < 1e-6             # (step + 1) / warmup_steps
    # shipped GPT-2 configuration: total_steps (default 1000) < warmup_steps (2000): the unsigned subtraction wraps,
    # progress is ~0 and the rate simply stays at the base rate after the warm-up
    o = _Opt(3e-4)
    s = S.WarmupCosineAnnealing(o, warmup_steps=2000, total_steps=1000, start_lr=0.0, eta_min=0.0)
    for _ in range(2500):
        s.step()
    assert abs(o.learning_rate - 3e-4) < 1e-8
    o = _Opt(1.0)
    s = S.ReduceLROnPlateau(o, mode="min", factor=0.1, patience=1)
    for m in (1.0, 1.0, 1.0, 1.0):
        s.step(m)
    assert o.learning_rate < 1.0
