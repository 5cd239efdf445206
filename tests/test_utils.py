

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
