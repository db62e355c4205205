"""Command-line utilities shipped with the framework (run as ``python -m torchtitan_b200.scripts.<name>``):
``loss_compare``, ``generate.test_generate``, ``checkpoint_conversion.convert_from_hf / convert_to_hf /
numerical_tests_example`` and ``download_hf_assets``."""
