from .bitsmoe_auto_patch import (build_patched_model, ensure_auto_patch_installed, patch_bitsmoe_inplace,  # noqa: F401
                                 prepare_bitsmoe_runtime)
