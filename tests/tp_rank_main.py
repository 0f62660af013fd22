"""One rank of the two-GPU tensor-parallel check (launched by tests/test_tp.py through
torch.distributed.run).  Every rank builds the same seeded model on the host, keeps its shard,
decodes greedily, and rank 0 compares with the oracle that adds shard partials in rank order."""
import json
import os
import sys
from dataclasses import replace

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ggml_type = int(sys.argv[1])
    allreduce = sys.argv[2] if len(sys.argv) > 2 else "p2p"
    rank, local_rank, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    os.environ["ADAM_B200_DEVICE"] = str(local_rank)
    import adam_b200 as A
    from adam_b200 import synth
    from adam_b200.config import GenerationConfig, tiny_gemma3
    from adam_b200.tp import ADAMEngineTP, shard_plan
    from oracle.decoder import OracleDecoder, dequant_model

    cfg = replace(tiny_gemma3(), n_layer=3, n_embd=256, n_head=4, n_head_kv=2, head_dim=128, head_dim_kv=128, n_ff=768, n_vocab=512)
    tensors = synth.build_model(cfg, ggml_type, seed=11)
    prompt = synth.random_prompt(cfg.n_vocab, 9, seed=4)
    n_gen = 12
    gpu = A.init()
    eng = ADAMEngineTP(gpu, cfg, tensors, rank, world, kv_cap=128, kv_dtype="f32", allreduce=allreduce)
    ar_used = eng._ar is not None
    toks, _ = eng.generate(prompt, GenerationConfig(max_tokens=n_gen, top_k=1, temperature=0.0, repeat_penalty=1.0, eos_token_ids=()))
    graph_used = bool(eng._graphs)
    # a prompt of more than one 64-row chunk: chunked prefill (all-reduces of 64 and 13 rows, then of
    # one row per decode step) against the same prompt consumed token by token
    long_prompt = list(map(int, synth.random_prompt(cfg.n_vocab, 78, seed=5)))
    long_toks, _ = eng.generate(long_prompt, GenerationConfig(max_tokens=6, top_k=1, temperature=0.0, repeat_penalty=1.0, eos_token_ids=()))
    eng.begin([long_prompt], [128])
    eng.prefill(len(long_prompt) - 1, chunked=False)
    by_token = []
    for _ in range(6):
        eng.step(1, lm_head=True)
        by_token.append(int(eng.read_state()[1][0]))
    # teacher-forced logits of this rank's vocabulary shard for the whole sequence
    seq = list(map(int, prompt)) + toks
    local_logits = eng.logits_trace(seq[:-1], direct=True)
    mine = torch.from_numpy(local_logits).cuda()
    gathered = [torch.empty_like(mine) for _ in range(world)]          # equal vocabulary shards in this configuration
    dist.all_gather(gathered, mine)
    logits = torch.cat(gathered, dim=1).cpu().numpy()
    err = gpu.device_error()
    eng.close()
    gpu.shutdown()
    if rank == 0:
        bounds = shard_plan(cfg, 0, world, ggml_type).ff_bounds
        dec = OracleDecoder(cfg, dequant_model(tensors), kv_cap=64, tp_size=world, tp_ff_bounds=bounds)
        ref_logits = np.stack([dec.forward(t, i) for i, t in enumerate(seq[:-1])])
        ref_ids = [int(r.argmax()) for r in ref_logits[len(prompt) - 1:]]
        rel = float(np.abs(logits - ref_logits).max() / np.abs(ref_logits).max())
        dec2 = OracleDecoder(cfg, dequant_model(tensors), kv_cap=128, tp_size=world, tp_ff_bounds=bounds)
        long_ref, seq2 = [], list(long_prompt)
        for i in range(len(long_prompt) + 5):
            lg = dec2.forward(seq2[i], i)
            if i >= len(long_prompt) - 1:
                long_ref.append(int(lg.argmax()))
                seq2.append(long_ref[-1])
        print(json.dumps({"ids_equal": toks == ref_ids, "tokens": toks, "ref": ref_ids, "logit_rel_err": rel,
                          "graph_used": graph_used,
                          "long_ids_equal": long_toks == long_ref, "long_equals_by_token": long_toks == by_token, "long": long_toks, "long_ref": long_ref, "long_by_token": by_token, "p2p_allreduce": ar_used, "device_error": int(err)}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
