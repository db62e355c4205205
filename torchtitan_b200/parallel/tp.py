"""placeholder"""
class _LP:
    enabled = False
LOSS_PARALLEL = _LP()
def apply_tp_to_decoder(*a, **k):
    raise NotImplementedError
