"""moc_b200: B200 (sm_100a) implementation of the Mixture-of-Channels sparse SwiGLU FFN.

Public surface = the FFN plugin surface of xiaohuangji/MoC (``moc/ffn.py``,
``moc/inference/inference_ffn.py``): ``build_ffn``, ``MoCSwiGLUFFN``, ``StandardSwiGLUFFN``,
``InferenceMoCSwiGLUFFN``, plus ``install_into`` to rebind the reference package's factory.
"""
from .ffn import (  # noqa: F401
    MoCSwiGLUFFN,
    StandardSwiGLUFFN,
    build_ffn,
    install_into,
    set_grad_ready_hook,
    set_status_checks,
)
from ._lib import flush_status  # noqa: F401

__all__ = [
    "MoCSwiGLUFFN",
    "StandardSwiGLUFFN",
    "build_ffn",
    "install_into",
    "set_grad_ready_hook",
    "set_status_checks",
    "flush_status",
]


def __getattr__(name):
    if name == "InferenceMoCSwiGLUFFN":
        from .inference import InferenceMoCSwiGLUFFN
        return InferenceMoCSwiGLUFFN
    raise AttributeError(name)
