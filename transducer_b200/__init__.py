"""transducer_b200: sm_100a RNN-T loss and Viterbi for an additive joiner.

Drop-in for the CUDA path of awni/transducer (transducer/__init__.py:1 exports the
same single name)."""
from .torch_binding import TransducerLoss
from .host_pipeline import HostLossPipeline

__all__ = ["TransducerLoss", "HostLossPipeline"]
