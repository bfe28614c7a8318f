"""Pipeline-parallel send/recv: never take the "send a slice, all-gather on the receiver" shortcut.

Upstream shards PP activations over the TP group and re-assembles them with an all-gather on the
receiving stage.  With NVSwitch the full tensor crosses at link rate and the extra TP all-gather
(one more launch + barrier per micro-batch) costs more than it saves, and the fused row-parallel
kernels already leave the activation replicated.  Off unless B200_PP_DISABLE_ALLGATHER=1.
Parity: vllm_metax/patch/bugfix/deepseek_v4/parallel_state.py:12-20.
"""
from .. import utils
from ... import envs


@utils.patch("vllm.distributed.parallel_state", "GroupCoordinator._should_use_all_gather", allow_new=True,
             when=lambda: bool(envs.B200_PP_DISABLE_ALLGATHER))
def _should_use_all_gather(self, *args, **kwargs) -> bool:
    return False
