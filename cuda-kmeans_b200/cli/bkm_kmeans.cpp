/*
 * bkm-kmeans - command-line harness for libbkm with the flag names, units and output format of
 * the k-means executable of krulis-martin/cuda-kmeans (experimental/k-means/k-means/k-means.cpp:
 * arguments :297-330, timing and output :149-169, verification :171-182), so that experiment
 * scripts written for that executable can drive the B200 library unchanged:
 *
 *   bkm-kmeans --N 2M --dim 32 --k 1024 --iterations 20 --layout soa --algorithm b200 --verify
 *
 * stdout: "<ms per iteration> <ns per input float>"; progress messages go to stderr.
 * Algorithms: b200 (automatic variants), b200_exact, b200_simt, b200_tc, serial (the built-in
 * single-thread check, small sizes only).  Flags that tune the reference's own kernels
 * (--cudaBlockSize, --cudaBlockCount, --cudaSharedMemorySize, --privatizedCopies,
 * --itemsPerThread, --regsCache) are accepted and ignored; --Rscript is refused; --double runs the
 * library's fp64 path (reference arithmetic in double; one GPU).
 * The inputs are the reference executable's own for the same --N --k --dim --seed --layout
 * (reference_data.hpp restates its generator call for call); without --seed the reference draws a
 * random seed, this harness uses 42.  --dumpInputs <file> writes them out (with --dryRun: and stops).
 * --gpus G (not in the reference, which drives device 0 only) shards the points over G GPUs.
 */
#include "bkm.h"
#include "reference_data.hpp"

#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <numeric>
#include <random>
#include <stdexcept>
#include <string>
#include <vector>

namespace {

struct Options {
	uint64_t n = 10240;
	uint32_t k = 128, dim = 20, iterations = 1, seed = 42, gpus = 1;
	bool assignment_only = false, verify = false, dry_run = false, use_double = false;
	std::string algorithm = "b200", layout = "aos", layout_means, dump_inputs;
};

[[noreturn]] void usage_error(const std::string& what)
{
	std::cout << "Invalid arguments: " << what << std::endl << std::endl
		<< "Usage: bkm-kmeans [--N n] [--k k] [--dim d] [--iterations i | --assignmentOnly] [--seed s]\n"
		<< "                  [--algorithm b200|b200_exact|b200_simt|b200_tc|serial] [--layout aos|soa]\n"
		<< "                  [--layoutMeans aos|soa] [--verify] [--dryRun] [--dumpInputs file] [--gpus g] [--double]\n"
		<< "Integers take the suffixes k, M, G (powers of 1024)." << std::endl;
	std::exit(1);
}

// "2M" -> 2097152: the suffixes of the reference's integer arguments
uint64_t parse_int(const std::string& name, const std::string& text)
{
	if (text.empty()) usage_error("--" + name + " needs a value");
	size_t pos = 0;
	unsigned long long v = 0;
	try { v = std::stoull(text, &pos); } catch (...) { usage_error("--" + name + ": '" + text + "' is not a number"); }
	uint64_t mult = 1;
	if (pos < text.size()) {
		const std::string suffix = text.substr(pos);
		if (suffix == "k") mult = 1024ull;
		else if (suffix == "M") mult = 1024ull * 1024;
		else if (suffix == "G") mult = 1024ull * 1024 * 1024;
		else usage_error("--" + name + ": unknown suffix '" + suffix + "'");
	}
	return (uint64_t)v * mult;
}

Options parse(int argc, char** argv)
{
	Options o;
	bool iterations_given = false;
	for (int i = 1; i < argc; ++i) {
		std::string a = argv[i];
		if (a.rfind("--", 0) != 0) usage_error("unexpected argument '" + a + "'");
		a = a.substr(2);
		auto value = [&]() -> std::string {
			if (i + 1 >= argc) usage_error("--" + a + " needs a value");
			return argv[++i];
		};
		if (a == "N") o.n = parse_int(a, value());
		else if (a == "k") o.k = (uint32_t)parse_int(a, value());
		else if (a == "dim") o.dim = (uint32_t)parse_int(a, value());
		else if (a == "iterations") { o.iterations = (uint32_t)parse_int(a, value()); iterations_given = true; }
		else if (a == "seed") o.seed = (uint32_t)parse_int(a, value());
		else if (a == "assignmentOnly") o.assignment_only = true;
		else if (a == "verify") o.verify = true;
		else if (a == "dryRun") o.dry_run = true;
		else if (a == "algorithm") o.algorithm = value();
		else if (a == "layout") o.layout = value();
		else if (a == "layoutMeans") o.layout_means = value();
		else if (a == "dumpInputs") o.dump_inputs = value();
		else if (a == "gpus") o.gpus = (uint32_t)parse_int(a, value());
		else if (a == "cudaBlockSize" || a == "cudaBlockCount" || a == "cudaSharedMemorySize" || a == "privatizedCopies" ||
			a == "itemsPerThread" || a == "regsCache") (void)value();
		else if (a == "double") o.use_double = true;
		else if (a == "Rscript") usage_error("--Rscript is not supported");
		else usage_error("unknown argument '--" + a + "'");
	}
	if (o.layout_means.empty()) o.layout_means = o.layout;
	if (o.assignment_only && iterations_given) usage_error("--assignmentOnly conflicts with --iterations");
	if (o.dim < 1 || o.k < 1 || o.n < 1 || o.iterations < 1) usage_error("N, k, dim and iterations must be positive");
	if (o.gpus < 1 || o.gpus > 8) usage_error("--gpus must be 1..8");
	if (o.gpus > 1 && o.assignment_only) usage_error("--assignmentOnly runs on one GPU");
	if (o.use_double && o.gpus > 1) usage_error("--double runs on one GPU");
	for (const std::string* l : {&o.layout, &o.layout_means})
		if (*l != "aos" && *l != "soa") usage_error("layout must be aos or soa");
	return o;
}

inline size_t at(bool soa, uint64_t i, uint32_t j, uint64_t rows, uint32_t dim) { return soa ? (size_t)j * rows + i : (size_t)i * dim + j; }

// The reference executable's inputs for these arguments (k-means.cpp:205-210): see reference_data.hpp.
template<typename F>
void generate(const Options& o, bool soa, bool soa_means, std::vector<F>& data, std::vector<F>& means)
{
	refdata::clustered_points(data, o.n, o.k, o.dim, o.seed, soa);
	refdata::shuffled_means(data, means, o.n, o.k, o.dim, o.seed, soa, soa_means);
}

// Raw dump of the generated inputs (for comparing them with the reference's): three 64-bit
// integers n, k, dim, then the data and the initial means as 32-bit floats in their layouts.
template<typename F>
void dump_inputs(const std::string& path, const Options& o, const std::vector<F>& data, const std::vector<F>& means)
{
	FILE* f = std::fopen(path.c_str(), "wb");
	if (!f) throw std::runtime_error("cannot open '" + path + "' for writing");
	const uint64_t head[3] = {o.n, o.k, o.dim};
	bool ok = std::fwrite(head, sizeof(head), 1, f) == 1 && std::fwrite(data.data(), sizeof(F), data.size(), f) == data.size() &&
		std::fwrite(means.data(), sizeof(F), means.size(), f) == means.size();
	ok = std::fclose(f) == 0 && ok;
	if (!ok) throw std::runtime_error("writing '" + path + "' failed");
}

// Single-thread Lloyd iterations with the semantics of the reference's serial algorithm
// (serial.hpp:21-96): Euclidean distance summed in dimension order, lowest index wins ties, an
// empty cluster gets the zero vector.  Used by --verify and --algorithm serial.
template<typename F>
void serial_kmeans(const Options& o, bool soa, bool soa_means, const std::vector<F>& data, std::vector<F> means,
	uint32_t iters, std::vector<F>& means_out, std::vector<uint32_t>& asg)
{
	asg.assign(o.n, 0);
	std::vector<uint32_t> counts(o.k);
	for (uint32_t it = 0; it < iters; ++it) {
		for (uint64_t i = 0; i < o.n; ++i) {
			uint32_t best = 0;
			F best_d = (F)0;
			for (uint32_t m = 0; m < o.k; ++m) {
				F sum = (F)0;
				for (uint32_t j = 0; j < o.dim; ++j) {
					const F diff = data[at(soa, i, j, o.n, o.dim)] - means[at(soa_means, m, j, o.k, o.dim)];
					sum += diff * diff;
				}
				const F dist = std::sqrt(sum);
				if (m == 0 || best_d > dist) { best_d = dist; best = m; }
			}
			asg[i] = best;
		}
		std::fill(means.begin(), means.end(), (F)0);
		std::fill(counts.begin(), counts.end(), 0u);
		for (uint64_t i = 0; i < o.n; ++i) {
			++counts[asg[i]];
			for (uint32_t j = 0; j < o.dim; ++j) means[at(soa_means, asg[i], j, o.k, o.dim)] += data[at(soa, i, j, o.n, o.dim)];
		}
		for (uint32_t m = 0; m < o.k; ++m)
			if (counts[m])
				for (uint32_t j = 0; j < o.dim; ++j) means[at(soa_means, m, j, o.k, o.dim)] /= (F)counts[m];
	}
	means_out = means;
}

void check(int rc)
{
	if (rc != BKM_OK) throw std::runtime_error(bkm_last_error());
}

double now_ms()
{
	return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// --double: the whole job in fp64 (k-means.cpp:340-345 runs every algorithm with F = double then).  The
// library has one fp64 path (reference arithmetic in double, bkm_kmeans_host_f64); the variant names
// that select fp32 kernels all map to it.  The timed region includes the copies to and from the GPU.
int run_double(const Options& o, bool soa, bool soa_means)
{
	std::vector<double> data, means, got_means;
	std::vector<uint32_t> got_asg;
	std::cerr << "Generating input data (" << o.n << " x " << o.dim << ") ..." << std::endl;
	std::cerr << "Seed is set to " << o.seed << std::endl;
	generate(o, soa, soa_means, data, means);
	if (!o.dump_inputs.empty()) {
		dump_inputs(o.dump_inputs, o, data, means);
		if (o.dry_run) return 0;
	}
	const uint32_t iters = o.assignment_only ? 1u : o.iterations;
	std::cerr << "Initializing ... 0 ms" << std::endl;
	std::cerr << "Running (" << iters << " iterations) ... ";
	double run_ms = 0.0;
	if (o.algorithm == "serial") {
		const double t0 = now_ms();
		serial_kmeans(o, soa, soa_means, data, means, iters, got_means, got_asg);
		run_ms = now_ms() - t0;
	} else {
		got_means = means;
		got_asg.resize(o.n);
		const double t0 = now_ms();
		check(bkm_kmeans_host_f64(data.data(), got_means.data(), got_asg.data(), o.n, o.k, o.dim, iters,
			soa ? BKM_LAYOUT_SOA : BKM_LAYOUT_AOS, soa_means ? BKM_LAYOUT_SOA : BKM_LAYOUT_AOS, 0));
		run_ms = now_ms() - t0;
	}
	std::cout << run_ms / (double)iters;
	std::cerr << " ms/iter (which is";
	std::cout << " " << (run_ms * 1000000.0 / ((double)iters * o.dim * (double)o.n));
	std::cerr << " ns/input float)";
	std::cout << std::endl;
	if (o.verify && o.algorithm != "serial") {
		std::cerr << "Verifying results ... ";
		std::vector<double> want_means;
		std::vector<uint32_t> want_asg;
		serial_kmeans(o, soa, soa_means, data, means, iters, want_means, want_asg);
		uint64_t errors = 0;
		for (uint64_t i = 0; i < o.n; ++i) errors += got_asg[i] != want_asg[i];
		if (!o.assignment_only) {
			double total = 0.0;
			for (uint32_t m = 0; m < o.k; ++m) {
				double d2 = 0.0;
				for (uint32_t j = 0; j < o.dim; ++j) {
					const double d = got_means[at(soa_means, m, j, o.k, o.dim)] - want_means[at(soa_means, m, j, o.k, o.dim)];
					d2 += d * d;
				}
				const double dist = std::sqrt(d2);
				total += dist;
				if (dist > 0.1) ++errors;
			}
			if (total / o.k > 0.01) ++errors;
		}
		std::cerr << (errors == 0 ? "OK" : "FAILED") << std::endl;
		if (errors) return 3;
	}
	return 0;
}

int run(const Options& o)
{
	const bool soa = o.layout == "soa", soa_means = o.layout_means == "soa";
	int variant = BKM_ASSIGN_AUTO;
	if (o.algorithm == "b200") variant = BKM_ASSIGN_AUTO;
	else if (o.algorithm == "b200_exact") variant = BKM_ASSIGN_EXACT;
	else if (o.algorithm == "b200_simt") variant = BKM_ASSIGN_SIMT;
	else if (o.algorithm == "b200_tc") variant = BKM_ASSIGN_TC;
	else if (o.algorithm != "serial") throw std::runtime_error("Unkown algorithm '" + o.algorithm + "'.");
	std::cerr << "Selected k-means algorithm: " << o.algorithm << std::endl;
	if (o.dry_run && o.dump_inputs.empty()) {
		std::cout << "N=" << o.n << " k=" << o.k << " dim=" << o.dim << " iterations=" << o.iterations << " seed=" << o.seed
			<< " layout=" << o.layout << " layoutMeans=" << o.layout_means << " assignmentOnly=" << o.assignment_only
			<< " verify=" << o.verify << std::endl;
		return 0;
	}

	if (o.use_double) return run_double(o, soa, soa_means);
	std::vector<float> data, means, got_means;
	std::vector<uint32_t> got_asg;
	std::cerr << "Generating input data (" << o.n << " x " << o.dim << ") ..." << std::endl;
	std::cerr << "Seed is set to " << o.seed << std::endl;
	generate(o, soa, soa_means, data, means);
	if (!o.dump_inputs.empty()) {
		dump_inputs(o.dump_inputs, o, data, means);
		if (o.dry_run) return 0;
	}
	uint32_t iters = o.iterations;
	double init_ms = 0.0, run_ms = 0.0;

	if (o.algorithm == "serial") {
		std::cerr << "Initializing ... 0 ms" << std::endl;
		std::cerr << "Running (" << iters << " iterations) ... ";
		const double t0 = now_ms();
		serial_kmeans(o, soa, soa_means, data, means, iters, got_means, got_asg);
		run_ms = now_ms() - t0;
	} else if (o.assignment_only) {
		// the assignment step alone on device buffers (the reference's --assignmentOnly micro-benchmark)
		std::cerr << "Initializing ... ";
		double t0 = now_ms();
		float *d_pts = nullptr, *d_means = nullptr;
		uint32_t* d_asg = nullptr;
		void* ws = nullptr;
		const size_t ws_bytes = bkm_workspace_bytes(o.n, o.k, o.dim);
		if (ws_bytes == 0) throw std::runtime_error("problem size not supported");
		if (cudaMalloc(&d_pts, data.size() * 4) != cudaSuccess || cudaMalloc(&d_means, means.size() * 4) != cudaSuccess ||
			cudaMalloc(&d_asg, o.n * 4) != cudaSuccess || cudaMalloc(&ws, ws_bytes) != cudaSuccess)
			throw std::runtime_error("cudaMalloc failed");
		cudaMemcpy(d_pts, data.data(), data.size() * 4, cudaMemcpyHostToDevice);
		cudaMemcpy(d_means, means.data(), means.size() * 4, cudaMemcpyHostToDevice);
		// untimed first call: one-off set-up inside the library
		check(bkm_assign_f32(d_pts, d_means, d_asg, o.n, o.k, o.dim, soa, soa_means, variant, ws, ws_bytes, nullptr));
		cudaDeviceSynchronize();
		init_ms = now_ms() - t0;
		std::cerr << init_ms << " ms" << std::endl;
		std::cerr << "Running (1 iterations) ... ";
		t0 = now_ms();
		check(bkm_assign_f32(d_pts, d_means, d_asg, o.n, o.k, o.dim, soa, soa_means, variant, ws, ws_bytes, nullptr));
		if (cudaDeviceSynchronize() != cudaSuccess) throw std::runtime_error("CUDA error after the assignment");
		run_ms = now_ms() - t0;
		check(bkm_workspace_check(ws, nullptr));
		got_asg.resize(o.n);
		cudaMemcpy(got_asg.data(), d_asg, o.n * 4, cudaMemcpyDeviceToHost);
		got_means = means;
		cudaFree(d_pts); cudaFree(d_means); cudaFree(d_asg); cudaFree(ws);
		iters = 1;
	} else {
		bkm_config_t cfg{};
		cfg.n = o.n; cfg.k = o.k; cfg.dim = o.dim;
		cfg.layout = soa ? BKM_LAYOUT_SOA : BKM_LAYOUT_AOS;
		cfg.layout_means = soa_means ? BKM_LAYOUT_SOA : BKM_LAYOUT_AOS;
		cfg.variant_assign = variant;
		cfg.num_gpus = (int32_t)o.gpus;          // > 1: the points are sharded over GPUs 0 .. gpus-1 of this process
		bkm_handle_t h = nullptr;
		std::cerr << "Initializing ... ";
		double t0 = now_ms();
		check(bkm_create(&cfg, &h));
		check(bkm_initialize(h, data.data(), means.data()));
		init_ms = now_ms() - t0;
		std::cerr << init_ms << " ms" << std::endl;
		std::cerr << "Running (" << iters << " iterations) ... ";
		t0 = now_ms();
		check(bkm_run(h, iters));
		run_ms = now_ms() - t0;
		got_means.resize(means.size());
		got_asg.resize(o.n);
		check(bkm_get_means(h, got_means.data()));
		check(bkm_get_assignment(h, got_asg.data()));
		bkm_destroy(h);
	}

	std::cout << run_ms / (double)iters;
	std::cerr << " ms/iter (which is";
	std::cout << " " << (run_ms * 1000000.0 / ((double)iters * o.dim * (double)o.n));
	std::cerr << " ns/input float)";
	std::cout << std::endl;

	if (o.verify && o.algorithm != "serial") {
		std::cerr << "Verifying results ... ";
		std::vector<float> want_means;
		std::vector<uint32_t> want_asg;
		// the assignment a run returns was computed against the means of the iteration before the last
		serial_kmeans(o, soa, soa_means, data, means, o.assignment_only ? 1 : iters, want_means, want_asg);
		uint64_t errors = 0;
		for (uint64_t i = 0; i < o.n; ++i) errors += got_asg[i] != want_asg[i];
		if (!o.assignment_only) {
			// the reference's own acceptance rule (data.hpp:160-202): every mean within 0.1, 0.01 on average
			double total = 0.0;
			for (uint32_t m = 0; m < o.k; ++m) {
				double d2 = 0.0;
				for (uint32_t j = 0; j < o.dim; ++j) {
					const double d = (double)got_means[at(soa_means, m, j, o.k, o.dim)] - want_means[at(soa_means, m, j, o.k, o.dim)];
					d2 += d * d;
				}
				const double dist = std::sqrt(d2);
				total += dist;
				if (dist > 0.1) ++errors;
			}
			if (total / o.k > 0.01) ++errors;
		}
		std::cerr << (errors == 0 ? "OK" : "FAILED") << std::endl;
		if (errors) return 3;
	}
	return 0;
}

} // namespace

int main(int argc, char** argv)
{
	const Options o = parse(argc, argv);
	try {
		return run(o);
	} catch (std::exception& e) {
		std::cout << "Error: " << e.what() << std::endl << std::endl;
		return 2;
	}
}
