"""A small, whole, single-GPU inference engine for the Llama-style toy decoder, written for B200.

Sub-packages, from a request's tokens to its next token:

* ``config``   typed model and engine configurations, the architecture registry
* ``weights``  safetensors by tensor name, the manifest check, the seeded random-weights mode
* ``parts``    norm, position encoding, mixer (attention), feed-forward and their arrangement
* ``models``   one module per architecture: configuration -> parts, layer order, tensor names
* ``cache``    paged key/value pools per layer group, block tables, prefix cache, state slots
* ``engine``   the step function, the scheduler, the generation loop, trace replay
* ``sampling`` greedy / temperature / nucleus sampling on the device
* ``ops``      bindings of the hand-written sm_100a kernels in ``csrc``
"""

__version__ = "0.1.0"
