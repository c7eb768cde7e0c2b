"""The bookkeeping of repeated launches (kernels.LayerReplay) without a GPU: which arguments are exchanged, by what."""
import pytest
import torch

from forge_b200 import kernels


class FakeLib:
    def forge_last_error(self):
        return b"it failed"


def make_entry(log, pointer_args, rc=0):
    def fn(*args):
        log.append(args)
        return rc
    e = kernels._Entry.__new__(kernels._Entry)
    e.lib, e.name, e.fn, e.pointer_args = FakeLib(), "fake_kernel", fn, tuple(pointer_args)
    return e


def test_pointers_into_the_layers_tensors_are_exchanged_and_nothing_else():
    w1, b1, c1 = torch.zeros(64), torch.zeros(8), torch.zeros(4, 16)
    w2, b2, c2 = torch.zeros(64), torch.zeros(8), torch.zeros(4, 16)
    other = torch.zeros(32)                                   # an intermediate: the same address in every layer
    log = []
    entry = make_entry(log, pointer_args=(0, 1, 2, 4))
    rec = kernels.record_launches()
    with rec:
        assert kernels._recording[0] is rec.calls
        # arguments: weight, a view 12 elements into the weight, an intermediate, a size, the cache + 128 bytes
        entry(w1.data_ptr(), w1.data_ptr() + 48, other.data_ptr(), 7, c1.data_ptr() + 128)
        entry(b1.data_ptr(), 0, None, w1.data_ptr(), 0)       # argument 3 is no pointer argument: left alone
        kernels.count_launches(2)
    assert kernels._recording[0] is None and len(rec.calls) == 2 and rec.launches == 2
    replay = kernels.LayerReplay(rec, [w1, b1, None, c1])
    del log[:]
    before = kernels.launch_count()
    replay.run([w2, b2, None, c2])
    assert kernels.launch_count() == before + 2
    assert log[0] == (w2.data_ptr(), w2.data_ptr() + 48, other.data_ptr(), 7, c2.data_ptr() + 128)
    assert log[1] == (b2.data_ptr(), 0, None, w1.data_ptr(), 0)
    # and again for a third layer: the recorded arguments are not used up
    w3, b3, c3 = torch.zeros(64), torch.zeros(8), torch.zeros(4, 16)
    del log[:]
    replay.run([w3, b3, None, c3])
    assert log[0][0] == w3.data_ptr() and log[0][4] == c3.data_ptr() + 128 and log[1][0] == b3.data_ptr()


def test_a_layer_with_other_optional_tensors_is_refused():
    w1, b1 = torch.zeros(16), torch.zeros(4)
    log = []
    entry = make_entry(log, pointer_args=(0,))
    with kernels.record_launches() as rec:
        entry(w1.data_ptr())
    replay = kernels.LayerReplay(rec, [w1, b1])
    with pytest.raises(kernels.KernelError, match="optional tensors"):
        replay.run([torch.zeros(16), None])


def test_a_failing_launch_raises_with_the_librarys_message():
    w1 = torch.zeros(16)
    ok_log, bad_log = [], []
    with kernels.record_launches() as rec:
        make_entry(ok_log, (0,))(w1.data_ptr())
        rec.calls.append((make_entry(bad_log, (0,), rc=3), (w1.data_ptr(),)))
    replay = kernels.LayerReplay(rec, [w1])
    with pytest.raises(kernels.KernelError, match="fake_kernel: it failed"):
        replay.run([torch.zeros(16)])


def test_parts_declare_it_only_for_exactly_the_stock_classes():
    from forge_b200.parts.base import Runtime, replay_of
    from forge_b200.parts.norm import RMSNorm
    rt = Runtime(torch.device("cpu"), torch.float32)
    n = RMSNorm(rt, 8, 1e-5)
    n.weight = torch.ones(8)
    key, tensors = replay_of(n)
    assert tensors == [n.weight] and key == ("rmsnorm", 8, 1e-5, torch.float32)

    class Mine(RMSNorm):
        pass
    m = Mine(rt, 8, 1e-5)
    m.weight = torch.ones(8)
    assert replay_of(m) is None
    assert replay_of(object()) is None


def test_launches_marked_once_per_step_are_left_out():
    """What the whole step shares is made inside the first layer that needs it: those launches are made, but
    neither noted nor counted for the layers that repeat the notes."""
    log = []
    entry = make_entry(log, pointer_args=(0,))
    w = torch.zeros(8)
    with kernels.record_launches() as rec:
        with kernels.once_per_step():
            kernels._check(FakeLib(), entry(w.data_ptr(), 1), "table")        # runs, is not noted
        kernels._check(FakeLib(), entry(w.data_ptr(), 2), "product")
    assert [a[1] for a in log] == [1, 2]
    assert len(rec.calls) == 1 and rec.calls[0][1][1] == 2 and rec.launches == 1
    assert kernels._once[0] == 0
