// b200-node: the managed-node side of the worker contract.
//
//   b200-node psionic attach --file attachment.json --state-dir DIR
//   b200-node psionic receipt append --state-dir DIR --assignment-id A --product-id P --worker-id W
//                                    --status succeeded|failed|refused --evidence-digest sha256:...
//                                    [--profile-digest sha256:...] [--receipt-id R]
//   b200-node status --json --state-dir DIR
//
// `attach` validates a worker-attachment document and stores it in the node state; `status`
// projects ready inference / training / sandbox workers into capability lanes (a crashed worker
// degrades only its own row); `receipt append` writes one execution receipt per line, each with a
// digest over its own fields.  Field names, schema versions and validation rules are those of
// crates/openagents-cloud-contract/src/lib.rs:11-12, 1724-1770 (types), 1772-1808 and 1811-1850
// (validation), and of the node commands at crates/oa-node/src/main.rs:69-70, 3796-3900.
#include <chrono>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <sstream>

#include "mini_json.h"

static const char* kAttachmentVersion = "openagents.psionic_worker_attachment.v1";
static const char* kReceiptVersion = "openagents.psionic_execution_receipt.v1";
static const char* kWorkersFile = "psionic-workers.json";
static const char* kReceiptsFile = "psionic-execution-receipts.jsonl";

static std::string read_file(const std::string& path, bool* ok) {
  std::ifstream f(path, std::ios::binary);
  *ok = (bool)f;
  std::stringstream ss;
  ss << f.rdbuf();
  return ss.str();
}

static bool blank(const std::string& s) { return s.find_first_not_of(" \t\r\n") == std::string::npos; }
static bool starts_with(const std::string& s, const char* p) { return s.rfind(p, 0) == 0; }

// Returns "" when the attachment is valid, else the reason.
static std::string validate_attachment(const mj::Value& v) {
  if (v.kind != mj::Value::Obj) return "attachment must be a JSON object";
  const mj::Value* sv = v.get("schema_version");
  if (!sv || !sv->is_str() || sv->str != kAttachmentVersion)
    return "unexpected psionic worker attachment version '" + (sv && sv->is_str() ? sv->str : std::string()) + "'";
  const mj::Value* up = v.get("updated_at_ms");
  if (!up || up->kind != mj::Value::Num) return "updated_at_ms must be a number";
  const mj::Value* ws = v.get("workers");
  if (!ws || ws->kind != mj::Value::Arr || ws->arr.empty()) return "psionic worker attachment must contain at least one worker";
  for (auto& wp : ws->arr) {
    const mj::Value& w = *wp;
    if (w.kind != mj::Value::Obj) return "worker must be an object";
    for (const char* field : {"product_id", "worker_id"}) {
      const mj::Value* x = w.get(field);
      if (!x || !x->is_str() || blank(x->str)) return std::string(field) + " must not be empty";
    }
    const std::string id = w.get("worker_id")->str;
    const mj::Value* kind = w.get("worker_kind");
    if (!kind || !kind->is_str() || (kind->str != "inference" && kind->str != "training" && kind->str != "sandbox"))
      return "psionic worker '" + id + "' has an unknown worker_kind";
    const mj::Value* ready = w.get("ready");
    const mj::Value* crashed = w.get("crashed");
    if (!ready || !ready->is_bool() || !crashed || !crashed->is_bool()) return "ready and crashed must be booleans";
    if (ready->b && crashed->b) return "psionic worker '" + id + "' cannot be both ready and crashed";
    const mj::Value* ev = w.get("evidence_digest");
    if (ev && ev->kind != mj::Value::Null && (!ev->is_str() || !starts_with(ev->str, "sha256:")))
      return "psionic worker '" + id + "' evidence_digest must be sha256";
  }
  return "";
}

static std::string arg(int argc, char** argv, const char* name, const char* dflt = "") {
  for (int i = 0; i + 1 < argc; i++)
    if (std::string(argv[i]) == name) return argv[i + 1];
  return dflt;
}
static bool flag(int argc, char** argv, const char* name) {
  for (int i = 0; i < argc; i++)
    if (std::string(argv[i]) == name) return true;
  return false;
}

static int cmd_attach(int argc, char** argv) {
  const std::string file = arg(argc, argv, "--file"), dir = arg(argc, argv, "--state-dir", ".");
  bool ok;
  const std::string text = read_file(file, &ok);
  if (!ok) {
    std::cerr << "cannot read " << file << "\n";
    return 2;
  }
  std::string err;
  mj::Ptr v = mj::parse(text, &err);
  if (!v) {
    std::cerr << "invalid JSON: " << err << "\n";
    return 2;
  }
  err = validate_attachment(*v);
  if (!err.empty()) {
    std::cerr << err << "\n";
    return 3;
  }
  std::string out;
  mj::write(*v, out);
  const std::string tmp = dir + "/" + kWorkersFile + ".tmp";
  {
    std::ofstream f(tmp, std::ios::binary);
    if (!f) {
      std::cerr << "cannot write state under " << dir << "\n";
      return 2;
    }
    f << out << "\n";
  }
  if (std::rename(tmp.c_str(), (dir + "/" + kWorkersFile).c_str()) != 0) return 2;
  std::cout << "{\"attached_workers\":" << v->get("workers")->arr.size() << ",\"attachment_digest\":\"sha256:"
            << mj::sha256_hex(out) << "\"}\n";
  return 0;
}

static int cmd_receipt_append(int argc, char** argv) {
  const std::string dir = arg(argc, argv, "--state-dir", ".");
  const std::string assignment = arg(argc, argv, "--assignment-id"), product = arg(argc, argv, "--product-id"),
                    worker = arg(argc, argv, "--worker-id"), status = arg(argc, argv, "--status"),
                    evidence = arg(argc, argv, "--evidence-digest"), profile = arg(argc, argv, "--profile-digest");
  for (auto& kv : {std::make_pair("assignment_id", assignment), std::make_pair("product_id", product),
                   std::make_pair("worker_id", worker), std::make_pair("psionic_evidence_digest", evidence)})
    if (blank(kv.second)) {
      std::cerr << kv.first << " must not be empty\n";
      return 3;
    }
  if (status != "succeeded" && status != "failed" && status != "refused") {
    std::cerr << "status must be succeeded, failed or refused\n";
    return 3;
  }
  if (!starts_with(evidence, "sha256:")) {
    std::cerr << "psionic_evidence_digest must be a sha256 digest reference\n";
    return 3;
  }
  if (!profile.empty() && !starts_with(profile, "sha256:")) {
    std::cerr << "profile_digest must be a sha256 digest reference\n";
    return 3;
  }
  if (starts_with(product, "sandbox.") && profile.empty()) {
    std::cerr << "sandbox execution receipts must cite profile_digest\n";
    return 3;
  }
  const std::string now_arg = arg(argc, argv, "--emitted-at-ms");
  const long long now = !now_arg.empty() ? std::atoll(now_arg.c_str())
                                         : std::chrono::duration_cast<std::chrono::milliseconds>(
                                               std::chrono::system_clock::now().time_since_epoch()).count();
  std::string body;   // the digest covers every field but itself, in this order
  auto field = [&](const char* k, const std::string& val, bool first = false) {
    if (!first) body.push_back(',');
    mj::escape(k, body);
    body.push_back(':');
    mj::escape(val, body);
  };
  field("schema_version", kReceiptVersion, true);
  std::string rid = arg(argc, argv, "--receipt-id");
  if (rid.empty()) rid = "psionic.receipt." + mj::sha256_hex(assignment + "|" + worker + "|" + std::to_string(now)).substr(0, 24);
  field("receipt_id", rid);
  field("assignment_id", assignment);
  field("product_id", product);
  field("worker_id", worker);
  field("status", status);
  if (!profile.empty()) field("profile_digest", profile);
  field("psionic_evidence_digest", evidence);
  const std::string digest = "sha256:" + mj::sha256_hex("{" + body + ",\"emitted_at_ms\":" + std::to_string(now) + "}");
  std::string line = "{" + body;
  line += ",\"receipt_digest\":";
  mj::escape(digest, line);
  line += ",\"emitted_at_ms\":" + std::to_string(now) + "}";
  std::ofstream f(dir + "/" + kReceiptsFile, std::ios::app | std::ios::binary);
  if (!f) {
    std::cerr << "cannot append under " << dir << "\n";
    return 2;
  }
  f << line << "\n";
  std::cout << line << "\n";
  return 0;
}

static int cmd_status(int argc, char** argv) {
  const std::string dir = arg(argc, argv, "--state-dir", ".");
  bool ok;
  std::string inf = "[", trn = "[", sbx = "[", workers = "[", receipts = "[";
  const std::string text = read_file(dir + "/" + kWorkersFile, &ok);
  bool attached = false;
  if (ok) {
    std::string err;
    mj::Ptr v = mj::parse(text, &err);
    if (v && validate_attachment(*v).empty()) {
      attached = true;
      for (auto& wp : v->get("workers")->arr) {
        const mj::Value& w = *wp;
        const bool ready = w.get("ready")->b && !w.get("crashed")->b;
        const std::string kind = w.get("worker_kind")->str;
        std::string row = "{\"worker_id\":";
        mj::escape(w.get("worker_id")->str, row);
        row += ",\"product_id\":";
        mj::escape(w.get("product_id")->str, row);
        row += ",\"worker_kind\":\"" + kind + "\",\"ready\":" + (ready ? "true" : "false") +
               ",\"crashed\":" + (w.get("crashed")->b ? "true" : "false") + "}";
        workers += (workers.size() > 1 ? "," : "") + row;
        if (ready) {
          std::string& lane = kind == "inference" ? inf : kind == "training" ? trn : sbx;
          if (lane.size() > 1) lane.push_back(',');
          mj::escape(w.get("product_id")->str, lane);
        }
      }
    }
  }
  const std::string rtext = read_file(dir + "/" + kReceiptsFile, &ok);
  size_t n_receipts = 0;
  if (ok) {
    std::istringstream ss(rtext);
    std::string line;
    while (std::getline(ss, line)) {
      if (blank(line)) continue;
      mj::Ptr r = mj::parse(line, nullptr);
      if (!r || r->kind != mj::Value::Obj) continue;
      const mj::Value* d = r->get("receipt_digest");
      if (!d || !d->is_str()) continue;
      if (n_receipts++) receipts.push_back(',');
      mj::escape(d->str, receipts);
    }
  }
  std::cout << "{\"psionic_attached\":" << (attached ? "true" : "false") << ",\"capabilities\":{\"inference_products\":" << inf
            << "],\"training_products\":" << trn << "],\"sandbox_profiles\":" << sbx << "]},\"psionic_workers\":" << workers
            << "],\"psionic_execution_receipt_digests\":" << receipts << "],\"psionic_execution_receipt_count\":" << n_receipts
            << "}\n";
  (void)flag;
  return 0;
}

int main(int argc, char** argv) {
  const std::string a1 = argc > 1 ? argv[1] : "", a2 = argc > 2 ? argv[2] : "", a3 = argc > 3 ? argv[3] : "";
  if (a1 == "psionic" && a2 == "attach") return cmd_attach(argc, argv);
  if (a1 == "psionic" && a2 == "receipt" && a3 == "append") return cmd_receipt_append(argc, argv);
  if (a1 == "status") return cmd_status(argc, argv);
  std::cerr << "usage: b200-node psionic attach --file F --state-dir D\n"
               "       b200-node psionic receipt append --state-dir D --assignment-id A --product-id P --worker-id W "
               "--status succeeded|failed|refused --evidence-digest sha256:... [--profile-digest sha256:...]\n"
               "       b200-node status --json --state-dir D\n";
  return 64;
}
