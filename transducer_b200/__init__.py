"""transducer_b200: sm_100a RNN-T loss and Viterbi for an additive joiner.

Drop-in for the CUDA path of awni/transducer (transducer/__init__.py:1 exports the
same single name).  The native library is loaded when one of the exported names is first
used, so helper modules that need no GPU (``transducer_b200.workloads``,
``transducer_b200.distributed``) can be imported by processes that must not load it."""

__all__ = ["TransducerLoss", "HostLossPipeline", "DeviceStatusError"]


def __getattr__(name):
    if name in ("TransducerLoss", "DeviceStatusError"):
        from . import torch_binding
        return getattr(torch_binding, name)
    if name == "HostLossPipeline":
        from .host_pipeline import HostLossPipeline
        return HostLossPipeline
    raise AttributeError("module %r has no attribute %r" % (__name__, name))
