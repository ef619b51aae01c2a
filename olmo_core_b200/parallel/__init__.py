"""
B200-native parallel runtime: the sharded-parameter engine (``fsdp``), tensor / sequence parallel layers
(``tensor``), context-parallel attention (``context``) and the symmetric peer-memory plumbing they share
(``symmetric``). Collective-shaped work runs inside CUDA kernels over NVLink peer pointers where a hot op
pairs compute with a collective; ``torch.distributed`` (NCCL / Gloo) is the control plane and the CPU path.
"""
