from bitsmoe_b200.models.base_mlp import BitsMoE_BaseMoeMLP


class BitsMoE_DeepSeekMLP(BitsMoE_BaseMoeMLP):
    """Packed expert container of the DeepSeek family (bitsmoe/models/deepseekv2/bitsmoe_mlp.py)."""
