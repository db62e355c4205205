"""placeholder"""
def apply_cp_to_attention_module(*a, **k):
    raise NotImplementedError
def prepare_context_parallel_input(*a, **k):
    raise NotImplementedError
