from .comm import Communicator, LoopbackGroup  # noqa: F401
