// nvfp4_shard: offline tensor-parallel repack of one NVFP4 MLP or of one layer's attention projections.
//
//   nvfp4_shard <in.safetensors> <out_prefix> <world> <gate_prefix> <up_prefix> <down_prefix>
//   nvfp4_shard attn <in.safetensors> <out_prefix> <world> <n_kv_heads> <q_prefix> <k_prefix> <v_prefix> <o_prefix>
//
// Reads <gate_prefix>/<up_prefix>/<down_prefix>.weight_packed|weight_scale|weight_global_scale from
// the checkpoint, merges gate and up by rows (as the reference does at load time,
// src/engine/model.cpp:456-514) and writes, for every rank r, <out_prefix>.rank<r>.safetensors with
//   gate_up.weight_packed [2I/P, H/2]   gate_up.weight_scale [2I/P, H/16]   gate_up.weight_global_scale
//   down.weight_packed    [H, Kp/2]     down.weight_scale    [H, Kp/16]     down.weight_global_scale
// Kp = I/P rounded up to a multiple of 256, the padding zero: the row and column split
// nvfp4_tp_mlp_create makes on the device (which then also interleaves the gate and up rows of its
// own copy in slabs of 16 for the fused SwiGLU epilogue; nvfp4_interleave_gate_up does that on the host).
// The attn form merges q, k and v by rows (src/engine/model.cpp:296-350), gives rank r its q rows and the
// k and v rows of its KV heads, and cuts the output projection by K like the down projection:
//   qkv.weight_packed [q/P + 2 kv_local, H/2]   qkv.weight_scale   qkv.weight_global_scale
//   o.weight_packed   [H, Kp/2]                 o.weight_scale     o.weight_global_scale
// the shards nvfp4_tp_attn_create cuts on the device.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/nvfp4_checkpoint.h"

static int fail(const char* what, int st) {
    std::fprintf(stderr, "nvfp4_shard: %s: %s\n", what, nvfp4_ckpt_status_string(st));
    return 1;
}

static nvfp4_ckpt_tensor tensor(const void* data, size_t nbytes, const char* dtype, long long d0, long long d1, int rank) {
    nvfp4_ckpt_tensor t{};
    t.data = data;
    t.nbytes = nbytes;
    std::snprintf(t.dtype, sizeof t.dtype, "%s", dtype);
    t.rank = rank;
    t.shape[0] = d0;
    t.shape[1] = d1;
    return t;
}

static int shard_attn(char** argv) {
    const int world = std::atoi(argv[4]), n_kv = std::atoi(argv[5]);
    nvfp4_ckpt* c = nullptr;
    if (int st = nvfp4_ckpt_open(argv[2], &c)) return fail(argv[2], st);
    nvfp4_host_weight parts[3], o;
    for (int i = 0; i < 3; ++i)
        if (int st = nvfp4_ckpt_linear(c, argv[6 + i], &parts[i])) return fail(argv[6 + i], st);
    if (int st = nvfp4_ckpt_linear(c, argv[9], &o)) return fail(argv[9], st);
    if (parts[1].N != parts[2].N) return fail("k and v rows differ", NVFP4_CKPT_E_SHAPE);
    const size_t rows_all = (size_t)parts[0].N + 2 * (size_t)parts[1].N, H = (size_t)parts[0].K;
    std::vector<uint8_t> mp(rows_all * H / 2), ms(rows_all * H / 16);
    nvfp4_host_weight merged;
    if (int st = nvfp4_merge_rows(parts, 3, mp.data(), ms.data(), &merged)) return fail("q/k/v merge", st);
    const int rows = nvfp4_tp_shard_qkv_rows(parts[0].N, parts[1].N, n_kv, world);
    if (rows < 0) return fail("qkv shard", rows);
    const int kp = nvfp4_tp_shard_down_k(o.K, world);
    if (kp < 0) return fail("o shard", kp);
    for (int r = 0; r < world; ++r) {
        std::vector<uint8_t> sp((size_t)rows * H / 2), ss((size_t)rows * H / 16), op((size_t)o.N * kp / 2), os((size_t)o.N * kp / 16);
        nvfp4_host_weight qs, osd;
        if (int st = nvfp4_tp_shard_qkv(&merged, parts[0].N, parts[1].N, n_kv, r, world, sp.data(), ss.data(), &qs)) return fail("qkv shard", st);
        if (int st = nvfp4_tp_shard_down(&o, r, world, op.data(), os.data(), &osd)) return fail("o shard", st);
        const char* names[6] = {"qkv.weight_packed", "qkv.weight_scale", "qkv.weight_global_scale",
                                "o.weight_packed", "o.weight_scale", "o.weight_global_scale"};
        const nvfp4_ckpt_tensor t[6] = {
            tensor(sp.data(), sp.size(), "U8", qs.N, qs.K / 2, 2), tensor(ss.data(), ss.size(), "F8_E4M3", qs.N, qs.K / 16, 2),
            tensor(&qs.global_scale, 4, "F32", 1, 0, 1),
            tensor(op.data(), op.size(), "U8", osd.N, osd.K / 2, 2), tensor(os.data(), os.size(), "F8_E4M3", osd.N, osd.K / 16, 2),
            tensor(&osd.global_scale, 4, "F32", 1, 0, 1)};
        const std::string out = std::string(argv[3]) + ".rank" + std::to_string(r) + ".safetensors";
        if (int st = nvfp4_ckpt_write(out.c_str(), names, t, 6)) return fail(out.c_str(), st);
        std::printf("%s: qkv [%d, %d], o [%d, %d (o_in/P = %d)]\n", out.c_str(), qs.N, qs.K, osd.N, osd.K, o.K / world);
    }
    nvfp4_ckpt_close(c);
    return 0;
}

int main(int argc, char** argv) {
    if (argc == 10 && !std::strcmp(argv[1], "attn")) return shard_attn(argv);
    if (argc != 7) {
        std::fprintf(stderr,
                     "usage: %s <in.safetensors> <out_prefix> <world> <gate_prefix> <up_prefix> <down_prefix>\n"
                     "       %s attn <in.safetensors> <out_prefix> <world> <n_kv_heads> <q_prefix> <k_prefix> <v_prefix> <o_prefix>\n",
                     argv[0], argv[0]);
        return 2;
    }
    const int world = std::atoi(argv[3]);
    nvfp4_ckpt* c = nullptr;
    if (int st = nvfp4_ckpt_open(argv[1], &c)) return fail(argv[1], st);
    nvfp4_host_weight parts[2], down;
    if (int st = nvfp4_ckpt_linear(c, argv[4], &parts[0])) return fail(argv[4], st);
    if (int st = nvfp4_ckpt_linear(c, argv[5], &parts[1])) return fail(argv[5], st);
    if (int st = nvfp4_ckpt_linear(c, argv[6], &down)) return fail(argv[6], st);
    const size_t gu_rows = (size_t)parts[0].N + (size_t)parts[1].N, H = (size_t)parts[0].K;
    std::vector<uint8_t> gu_p(gu_rows * H / 2), gu_s(gu_rows * H / 16);
    nvfp4_host_weight merged;
    if (int st = nvfp4_merge_rows(parts, 2, gu_p.data(), gu_s.data(), &merged)) return fail("gate/up merge", st);
    const int kp = nvfp4_tp_shard_down_k(down.K, world);
    if (kp < 0) return fail("down shard", kp);
    for (int r = 0; r < world; ++r) {
        const size_t rows = gu_rows / (size_t)world;
        std::vector<uint8_t> sp(rows * H / 2), ss(rows * H / 16), dp((size_t)down.N * kp / 2), ds((size_t)down.N * kp / 16);
        nvfp4_host_weight gs, dsrd;
        if (int st = nvfp4_tp_shard_gate_up(&merged, r, world, sp.data(), ss.data(), &gs)) return fail("gate_up shard", st);
        if (int st = nvfp4_tp_shard_down(&down, r, world, dp.data(), ds.data(), &dsrd)) return fail("down shard", st);
        const char* names[6] = {"gate_up.weight_packed", "gate_up.weight_scale", "gate_up.weight_global_scale",
                                "down.weight_packed", "down.weight_scale", "down.weight_global_scale"};
        const nvfp4_ckpt_tensor t[6] = {
            tensor(sp.data(), sp.size(), "U8", gs.N, gs.K / 2, 2), tensor(ss.data(), ss.size(), "F8_E4M3", gs.N, gs.K / 16, 2),
            tensor(&gs.global_scale, 4, "F32", 1, 0, 1),
            tensor(dp.data(), dp.size(), "U8", dsrd.N, dsrd.K / 2, 2), tensor(ds.data(), ds.size(), "F8_E4M3", dsrd.N, dsrd.K / 16, 2),
            tensor(&dsrd.global_scale, 4, "F32", 1, 0, 1)};
        const std::string out = std::string(argv[2]) + ".rank" + std::to_string(r) + ".safetensors";
        if (int st = nvfp4_ckpt_write(out.c_str(), names, t, 6)) return fail(out.c_str(), st);
        std::printf("%s: gate_up [%d, %d], down [%d, %d (I/P = %d)]\n", out.c_str(), gs.N, gs.K, dsrd.N, dsrd.K, down.K / world);
    }
    nvfp4_ckpt_close(c);
    return 0;
}
