

def test_step_profile_idle_gaps_from_a_fake_record():
    """Idle gaps are the intervals with no kernel of any stream running; overlapping kernels
    (two streams) extend the busy interval."""
    import torch

    from imfvideo_b200.utils.step_profile import idle_gaps

    class TR:
        def __init__(self, a, b):
            self.start, self.end = a, b

    class Ev:
        def __init__(self, name, a, b, cuda=True):
            self.name, self.time_range = name, TR(a, b)
            self.device_type = (torch.autograd.DeviceType.CUDA if cuda
                                else torch.autograd.DeviceType.CPU)

    class Prof:
        def events(self):
            return [Ev("k1", 0, 10), Ev("k2", 12, 20), Ev("side", 15, 40), Ev("k3", 30, 35),
                    Ev("cpu_op", 41, 49, cuda=False), Ev("k4", 50, 60)]

    gaps, idle = idle_gaps(Prof(), 5)
    assert idle == 2 + 10
    assert gaps[0] == (10, "side", "k4") and gaps[1] == (2, "k1", "k2")


def test_step_profile_launch_counts_from_a_fake_record():
    """Kernels are attributed to the torch op that launched them, grouped by op name and
    input shapes, most launches first; device events and ops without kernels are skipped."""
    from collections import namedtuple

    import torch

    from imfvideo_b200.utils.step_profile import launch_counts

    Kern = namedtuple("Kern", "name device duration")
    CPU, CUDA = torch.autograd.DeviceType.CPU, torch.autograd.DeviceType.CUDA

    class Ev:
        def __init__(self, name, shapes, kernels, dev=CPU):
            self.name, self.input_shapes, self.kernels, self.device_type = name, shapes, kernels, dev

    class Prof:
        def events(self):
            return [Ev("aten::add_", [[256], [256]], [Kern("add", 0, 2.0)]),
                    Ev("aten::add_", [[256], [256]], [Kern("add", 0, 3.0)]),
                    Ev("aten::mul", [[4, 4]], [Kern("mul", 0, 1.0), Kern("mul2", 0, 1.0),
                                               Kern("mul3", 0, 1.0)]),
                    Ev("aten::view", [[4, 4]], []),
                    Ev("add", [], [Kern("x", 0, 9.0)], dev=CUDA)]

    rows = launch_counts(Prof(), 5)
    assert rows == [(3, 3.0, "aten::mul", "[[4, 4]]"), (2, 5.0, "aten::add_", "[[256], [256]]")]
    assert launch_counts(Prof(), 1) == rows[:1]
