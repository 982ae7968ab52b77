"""`import fluidml` as with the reference's pybind11 module (src/python/pybind.cpp:23):
the same Executor factories, compile and invoke, running on the B200 back end."""
from fluidml_b200.executor import Executor  # noqa: F401
