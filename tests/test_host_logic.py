"""CPU tests of the host-side mirror: configuration validation, schedules, graph recording.  They read
like the reference's unit tests (cited) and need no GPU."""
import numpy as np
import pytest
import torch

from metal_candle_b200.graph import ComputationGraph, GraphNode, LazyTensor, NodeId, Operation
from metal_candle_b200.training import (AdamW, AdamWConfig, InvalidConfig, LoRAAdapterConfig, LoRAConfig, LRScheduler,
                                        TargetModule, TrainingConfig, TrainingStep)
from oracle import reference_ops as R


def test_lora_config_defaults_and_validation():
    # src/training/lora.rs:70-121
    c = LoRAConfig()
    assert (c.rank, c.alpha, c.dropout) == (8, 16.0, 0.0) and c.scaling() == 2.0
    for bad, msg in ((LoRAConfig(rank=0), "LoRA rank must be greater than 0"),
                     (LoRAConfig(alpha=0.0), "LoRA alpha must be positive"),
                     (LoRAConfig(dropout=1.0), r"LoRA dropout must be in \[0, 1\)")):
        with pytest.raises(InvalidConfig, match=msg):
            bad.validate()


def test_adapter_config_and_target_modules():
    # src/training/adapter.rs:33-62,96-124
    c = LoRAAdapterConfig()
    assert c.target_modules == [TargetModule.QProj, TargetModule.VProj]
    assert c.is_target(TargetModule.QProj) and not c.is_target(TargetModule.OProj)
    assert TargetModule.from_name("down_proj") is TargetModule.DownProj and TargetModule.from_name("nope") is None
    assert [m.value for m in TargetModule] == ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]
    assert c.to_lora_config().scaling() == 2.0


def test_adamw_config_validation():
    # src/training/optimizer.rs:51-107
    c = AdamWConfig()
    assert (c.learning_rate, c.beta1, c.beta2, c.epsilon, c.weight_decay) == (1e-4, 0.9, 0.999, 1e-8, 0.01)
    for kw, msg in ((dict(learning_rate=0.0), "learning rate must be positive"), (dict(beta1=1.0), "beta1 must be in"),
                    (dict(beta2=-0.1), "beta2 must be in"), (dict(epsilon=0.0), "epsilon must be positive"),
                    (dict(weight_decay=-1.0), "weight decay must be non-negative")):
        with pytest.raises(InvalidConfig, match=msg):
            AdamW(AdamWConfig(**kw))
    opt = AdamW()
    opt.set_lr(3e-4)
    assert opt.learning_rate() == 3e-4 and opt.step_count == 0
    with pytest.raises(Exception, match="not found in optimizer"):
        opt.step("missing", torch.zeros(2), torch.zeros(2))


def test_schedulers_match_oracle_and_reference_values():
    # src/training/scheduler.rs:312-373,401-419
    s = LRScheduler.linear(1000, 1e-3)
    assert s.get_lr(0) == 0.0 and abs(s.get_lr(500) - 5e-4) < 1e-7 and abs(s.get_lr(2000) - 1e-3) < 1e-9
    wc = LRScheduler.warmup_cosine(1000, 10_000, 1e-3, 1e-5)
    co = LRScheduler.cosine(10_000, 1e-3, 1e-5)
    for step in (0, 1, 499, 1000, 1001, 5000, 9999, 10_000, 20_000):
        assert wc.get_lr(step) == float(R.lr_warmup_cosine(step, 1000, 10_000, 1e-3, 1e-5))
        assert co.get_lr(step) == float(R.lr_cosine(step, 10_000, 1e-3, 1e-5))
    assert LRScheduler.constant(1e-4).get_lr(77) == float(np.float32(1e-4))
    LRScheduler.constant(1e-4).validate()
    for bad in (LRScheduler.constant(0.0), LRScheduler.linear(0, 1e-3), LRScheduler.cosine(0, 1e-3, 1e-5),
                LRScheduler.cosine(10, 1e-3, 1e-2), LRScheduler.warmup_cosine(10, 10, 1e-3, 1e-5)):
        with pytest.raises(InvalidConfig):
            bad.validate()


def test_training_config_defaults():
    # src/training/trainer.rs:30-39
    c = TrainingConfig()
    assert c.num_epochs == 3 and c.max_grad_norm == 1.0 and c.lr_scheduler.get_lr(5) == float(np.float32(1e-4))
    st = TrainingStep()
    assert st.step() == 0
    st.reset()
    assert st.step() == 0


def test_operation_names_shapes_and_arity_errors():
    # src/graph/operation.rs:53-166
    assert [Operation.Input().name(), Operation.Matmul().name(), Operation.Add().name(), Operation.Mul().name(),
            Operation.MulScalar(2.0).name(), Operation.LoRA(NodeId(1), NodeId(2), 2.0).name(),
            Operation.Softmax(1).name(), Operation.RMSNorm(1e-5).name()] == \
        ["input", "matmul", "add", "mul", "mul_scalar", "lora", "softmax", "rms_norm"]
    assert Operation.Matmul().output_shape([(2, 3), (3, 4)]) == (2, 4)
    assert Operation.Matmul().output_shape([(5, 2, 3), (3, 4)]) == (5, 2, 4)
    with pytest.raises(ValueError, match="Matmul requires 2 inputs, got 1"):
        Operation.Matmul().output_shape([(2, 3)])
    with pytest.raises(ValueError, match="Matmul dimension mismatch: 2×3 @ 4×5"):
        Operation.Matmul().output_shape([(2, 3), (4, 5)])
    with pytest.raises(ValueError, match="Matmul requires at least 2D tensors"):
        Operation.Matmul().output_shape([(3,), (3, 4)])
    with pytest.raises(ValueError, match="add requires 2 inputs, got 3"):
        Operation.Add().output_shape([(1,), (1,), (1,)])
    with pytest.raises(ValueError, match="Shape mismatch"):
        Operation.Mul().output_shape([(2, 2), (2, 3)])
    with pytest.raises(ValueError, match=r"LoRA requires 3 inputs \(input, a, b\), got 2"):
        Operation.LoRA(NodeId(0), NodeId(1), 1.0).output_shape([(2, 4), (4, 2)])
    # out_features comes from B (the reference returns the input shape here, which is wrong when out != in)
    assert Operation.LoRA(NodeId(0), NodeId(1), 1.0).output_shape([(2, 5, 16), (16, 4), (4, 32)]) == (2, 5, 32)
    with pytest.raises(ValueError, match="softmax requires 1 input, got 2"):
        Operation.Softmax(0).output_shape([(2,), (2,)])
    assert Operation.Softmax(0).output_dtype([torch.bfloat16]) == torch.bfloat16


def test_graph_recording_order_and_merge():
    # src/graph/node.rs:358-565; tests/lazy_execution.rs (graph shapes known before eval)
    a = LazyTensor.from_tensor(torch.ones(2, 3))
    b = a.add_tensor_to_graph(torch.ones(3, 4))
    c = a.matmul(b).mul_scalar(2.0)
    assert c.shape() == (2, 4) and c.dtype() == torch.float32 and c.graph_size() == 4 and not c.is_evaluated()
    assert a.is_evaluated() and a.node_id() == NodeId(0) and repr(c.node_id()) == "NodeId(3)"
    g = c._graph
    assert g.topological_order(c.node_id()) == [NodeId(0), NodeId(1), NodeId(2), NodeId(3)]
    with pytest.raises(ValueError, match=r"Input node NodeId\(9\) not found"):
        g.add_node(Operation.Add(), [NodeId(0), NodeId(9)])
    # operands from another graph are copied in with remapped ids
    other = LazyTensor.from_tensor(torch.ones(2, 4)).mul_scalar(3.0)
    d = c.add(other)
    assert d.graph_size() == 4 + 2 + 1 and d.shape() == (2, 4)
    order = g.topological_order(d.node_id())
    assert order[-1] == d.node_id() and len(order) == 7
    # a diamond is visited once
    e = d.add(d)
    assert len(g.topological_order(e.node_id())) == 8
    # a cycle (only constructible by hand) is reported
    g2 = ComputationGraph("cpu")
    g2.nodes.append(GraphNode(NodeId(0), Operation.MulScalar(1.0), [NodeId(1)], (1,), torch.float32))
    g2.nodes.append(GraphNode(NodeId(1), Operation.MulScalar(1.0), [NodeId(0)], (1,), torch.float32))
    with pytest.raises(ValueError, match="Circular dependency detected at node"):
        g2.topological_order(NodeId(0))
    with pytest.raises(Exception, match="Shape mismatch"):
        a.add(b)


def test_from_slice_and_constructors():
    t = LazyTensor.from_slice([1.0, 2.0, 3.0, 4.0], (2, 2), "cpu")
    assert t.shape() == (2, 2) and t.is_evaluated()
    assert LazyTensor.zeros((3,), torch.float32, "cpu").shape() == (3,)
    assert LazyTensor.ones((3, 2), torch.float32, "cpu").graph_size() == 1
    with pytest.raises(Exception):
        LazyTensor.from_slice([1.0, 2.0], (3,), "cpu")


def test_oracle_dropout_mask_is_a_pure_function_of_seed_and_position():
    """The restated mask of mcb_dropout: keep rate 1 - p, a call at offset k continues the stream of a call at offset 0,
    different seeds give different masks, p = 0 keeps everything; the LoRA training-mode forward scales kept entries
    of x A by 1 / (1 - p) (src/training/lora.rs:325-330 applies candle_nn::ops::dropout to the same tensor)."""
    import numpy as np

    from oracle import reference_ops as R

    whole = R.dropout_mask(100_000, 0.3, 7, 0)
    assert abs(whole.mean() - 0.7) < 5e-3
    assert np.array_equal(R.dropout_mask(1000, 0.3, 7, 5000), whole[5000:6000])
    assert not np.array_equal(R.dropout_mask(1000, 0.3, 8, 0), whole[:1000])
    assert R.dropout_mask(1000, 0.0, 7, 0).all()
    x = np.ones((4, 3)); A = np.ones((3, 2)); B = np.ones((2, 5))
    y = R.lora_forward_dropout(x, A, B, 2.0, 0.5, 11, 0)
    keep = R.dropout_mask(8, 0.5, 11, 0).reshape(4, 2)
    assert np.allclose(y, (np.where(keep, 3.0 / 0.5, 0.0) @ B) * 2.0)
