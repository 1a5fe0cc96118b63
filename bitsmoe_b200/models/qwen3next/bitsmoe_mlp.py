from bitsmoe_b200.models.base_mlp import BitsMoE_BaseMoeMLP


class BitsMoE_Qwen3NextMLP(BitsMoE_BaseMoeMLP):
    """Packed expert container of the Qwen3Next family (bitsmoe/models/qwen3next/bitsmoe_mlp.py)."""
