"""The Llama-architecture decoder on one GPU: linears on the tcgen05 kernels (through a single-rank communicator) against
the same model on torch.matmul."""
import pytest
import torch

pytestmark = pytest.mark.gpu


class _NoComm:
    """Single-rank stand-in that routes every linear to torch.matmul."""
    size, rank, fused = 1, 0, False

    def all_gather(self, send, recv, stream=None):
        recv.copy_(send.reshape(recv.shape))

    def reduce_scatter(self, send, recv, op=None, stream=None):
        recv.copy_(send.reshape(recv.shape))

    def all_reduce(self, send, recv=None, op=None, stream=None):
        if recv is not None and recv.data_ptr() != send.data_ptr():
            recv.copy_(send)

    def synchronize(self):
        pass


def test_tiny_llama_matches_torch_matmul_reference():
    from hccl_b200.comm import Communicator, get_root_info
    from hccl_b200.models.llama import Llama, LlamaConfig
    from hccl_b200.ops import gemm
    from hccl_b200.parallel import tensor_parallel

    cfg = LlamaConfig.tiny(vocab=512, hidden=256, layers=2, heads=8, kv_heads=4, ffn=512)
    tok = torch.randint(0, cfg.vocab_size, (2, 129), device="cuda", generator=torch.Generator(device="cuda").manual_seed(5))
    comm = Communicator.from_root_info(1, get_root_info(), 0)
    try:
        ours = Llama(cfg, comm, dtype=torch.bfloat16, device="cuda", seed=3)
        loss = ours(tok[:, :-1], tok[:, 1:].contiguous())
        loss.backward()
        torch.cuda.synchronize()
        gemm.check_error()
        tensor_parallel.use_native_gemm(False)
        ref = Llama(cfg, _NoComm(), dtype=torch.bfloat16, device="cuda", seed=3)
        rloss = ref(tok[:, :-1], tok[:, 1:].contiguous())
        rloss.backward()
        torch.cuda.synchronize()
    finally:
        tensor_parallel.use_native_gemm(True)
        comm.destroy()
    assert abs(loss.item() - rloss.item()) < 2e-2
    for (n1, p1), (n2, p2) in zip(ours.named_parameters(), ref.named_parameters()):
        a, b = p1.grad.float(), p2.grad.float()
        assert (a - b).abs().max().item() <= 5e-2 * (b.abs().max().item() + 1e-3), n1
