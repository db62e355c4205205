"""placeholder"""
def pipeline_llm(*a, **k):
    raise NotImplementedError
