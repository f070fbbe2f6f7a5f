"""A small, whole inference engine for one B200: from a model folder
(config.json, model.safetensors) to next tokens.

Sub-packages: `config` (typed configurations and the architecture registry),
`weights` (safetensors by tensor name, random-weight folders), `parts` (norms,
position encodings, mixers, feed-forwards, blocks), `models` (architectures as
layer plans), `cache` (paged keys/values, block tables, state slots), `engine`
(the step function, scheduler, entry points), `sampling`, `csrc` (the CUDA
kernels for sm_100a and their bindings).
"""
__version__ = "0.1.0"
