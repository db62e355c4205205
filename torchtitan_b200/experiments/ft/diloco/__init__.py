from .utils import fragment_llm, module_split

__all__ = ["fragment_llm", "module_split"]
