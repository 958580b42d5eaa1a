/*
 * EmitGolden.java — golden-vector emitter for the parse / validate / re-serialise path.
 *
 * UNCOMPILED HERE: this image has no JDK, no Gradle and no network, so this file has never been
 * compiled or run by the authors of this repository. It is shipped as source for a maintainer of
 * altro3/micronaut3-bug, who has all three.
 *
 * What it does: it drives the very calls that libpetjson.so replaces —
 *   io.micronaut.serde.ObjectMapper#readValue   (src/main/java/com/micronaut/bug/config/MyEntityConfig.java:34)
 *   ObjectMapper.getDefault()                   (src/main/java/com/micronaut/bug/service/MyEntityService.java:45)
 *   ObjectMapper#writeValueAsBytes              (what the response encoder of
 *                                                src/main/java/com/micronaut/bug/controller/MyEntityController.java:48-51 ends in)
 * — over the known-answer inputs of this repository and writes down what the real library answers:
 * for every record either the decoded value (re-serialised, so field order, number formatting and
 * escaping are visible) or the exception class, message and, where Jackson reports one, byte offset.
 *
 * How to run it (inside the reference project, which already has micronaut-serde-jackson on the
 * class path, build.gradle:89,104):
 *   1. python tests/golden/export_kat_inputs.py > kat_inputs.jsonl          (in this repository)
 *   2. copy this file to src/main/java/com/micronaut/bug/golden/EmitGolden.java, add
 *      `annotationProcessor("io.micronaut.serde:micronaut-serde-processor")` if it is not active,
 *      and run its main() with two arguments: kat_inputs.jsonl java_golden.jsonl
 *   3. copy java_golden.jsonl to tests/golden/ of this repository; tests/test_oracle_kat.py then
 *      checks the CPU checker (and through it the CUDA path) against it.
 *
 * The model classes below mirror petstore.json:823-972 and are annotated the way the reference
 * annotates its own types: @Serdeable as on api/EnumParam.java:15, @Introspected records with
 * @Nullable members as on config/data/ConfigData.java:15-30, enums mapped by value with
 * @JsonValue / @JsonCreator as on api/EnumParam.java:16-34 and config/data/VariantEnum.java:34-47.
 * Both of the tree's conventions for an unknown enum value are emitted (STRICT throws as
 * VariantEnum.byId does, LENIENT answers null as EnumParam.fromValue does): the line says which.
 */
package com.micronaut.bug.golden;

import com.fasterxml.jackson.annotation.JsonCreator;
import com.fasterxml.jackson.annotation.JsonValue;
import io.micronaut.core.annotation.Introspected;
import io.micronaut.core.annotation.Nullable;
import io.micronaut.core.type.Argument;
import io.micronaut.serde.ObjectMapper;
import io.micronaut.serde.annotation.Serdeable;

import java.io.BufferedReader;
import java.io.PrintWriter;
import java.nio.charset.StandardCharsets;
import java.nio.file.Files;
import java.nio.file.Path;
import java.time.OffsetDateTime;
import java.util.ArrayList;
import java.util.Base64;
import java.util.LinkedHashMap;
import java.util.List;
import java.util.Map;

public final class EmitGolden {

    /* ---- models: petstore.json:823-972, property order as in the specification ---- */
    @Serdeable
    public enum PetStatus {
        AVAILABLE("available"), PENDING("pending"), SOLD("sold");
        private final String value;
        PetStatus(String v) { value = v; }
        @JsonValue public String getValue() { return value; }
        @JsonCreator public static PetStatus fromValue(String v) {
            for (PetStatus s : values()) if (s.value.equals(v)) return s;
            throw new IllegalArgumentException("Unexpected value '" + v + "'");
        }
    }

    @Serdeable
    public enum PetStatusLenient {
        AVAILABLE("available"), PENDING("pending"), SOLD("sold");
        private final String value;
        PetStatusLenient(String v) { value = v; }
        @JsonValue public String getValue() { return value; }
        @JsonCreator public static PetStatusLenient fromValue(String v) {
            for (PetStatusLenient s : values()) if (s.value.equals(v)) return s;
            return null;
        }
    }

    @Serdeable
    public enum OrderStatus {
        PLACED("placed"), APPROVED("approved"), DELIVERED("delivered");
        private final String value;
        OrderStatus(String v) { value = v; }
        @JsonValue public String getValue() { return value; }
        @JsonCreator public static OrderStatus fromValue(String v) {
            for (OrderStatus s : values()) if (s.value.equals(v)) return s;
            throw new IllegalArgumentException("Unexpected value '" + v + "'");
        }
    }

    @Serdeable @Introspected
    public record Category(@Nullable Long id, @Nullable String name) { }

    @Serdeable @Introspected
    public record Tag(@Nullable Long id, @Nullable String name) { }

    /* name and photoUrls are required (petstore.json:873-876): no @Nullable */
    @Serdeable @Introspected
    public record Pet(@Nullable Long id, @Nullable Category category, String name, List<String> photoUrls,
                      @Nullable List<Tag> tags, @Nullable PetStatus status) { }

    @Serdeable @Introspected
    public record PetLenient(@Nullable Long id, @Nullable Category category, String name, List<String> photoUrls,
                             @Nullable List<Tag> tags, @Nullable PetStatusLenient status) { }

    @Serdeable @Introspected
    public record Order(@Nullable Long id, @Nullable Long petId, @Nullable Integer quantity, @Nullable OffsetDateTime shipDate,
                        @Nullable OrderStatus status, @Nullable Boolean complete) { }

    @Serdeable @Introspected
    public record User(@Nullable Long id, @Nullable String username, @Nullable String firstName, @Nullable String lastName,
                       @Nullable String email, @Nullable String password, @Nullable String phone, @Nullable Integer userStatus) { }

    private static Class<?> modelOf(String schema, boolean lenient) {
        switch (schema) {
            case "pet": return lenient ? PetLenient.class : Pet.class;
            case "order": return Order.class;
            case "user": return User.class;
            default: return null; /* "mixed": the reference has no discriminator for it; not emitted */
        }
    }

    /* ---- one record through the real mapper ---- */
    private static Map<String, Object> one(ObjectMapper mapper, byte[] bytes, Class<?> model) {
        Map<String, Object> r = new LinkedHashMap<>();
        try {
            Object v = mapper.readValue(bytes, Argument.of(model));
            r.put("ok", true);
            r.put("rewritten_b64", Base64.getEncoder().encodeToString(mapper.writeValueAsBytes(v)));
        } catch (Throwable t) {
            r.put("ok", false);
            Throwable root = t;
            while (root.getCause() != null && root.getCause() != root) root = root.getCause();
            r.put("exception", t.getClass().getName());
            r.put("root", root.getClass().getName());
            r.put("message", String.valueOf(t.getMessage()));
            /* Jackson's parse failures carry a location; validation failures of the decoder do not */
            for (Throwable c = t; c != null; c = c.getCause()) {
                if (c instanceof com.fasterxml.jackson.core.JsonProcessingException jpe && jpe.getLocation() != null) {
                    r.put("byte_offset", jpe.getLocation().getByteOffset());
                    break;
                }
                if (c.getCause() == c) break;
            }
        }
        return r;
    }

    /* NDJSON as this repository defines it: one readValue per LF-delimited line, blank lines skipped */
    private static List<byte[]> lines(byte[] in) {
        List<byte[]> out = new ArrayList<>();
        int s = 0;
        for (int i = 0; i <= in.length; i++) {
            if (i == in.length || in[i] == '\n') {
                boolean blank = true;
                for (int k = s; k < i; k++) if (in[k] != ' ' && in[k] != '\t' && in[k] != '\r') { blank = false; break; }
                if (!blank) out.add(java.util.Arrays.copyOfRange(in, s, i));
                s = i + 1;
            }
        }
        return out;
    }

    public static void main(String[] args) throws Exception {
        ObjectMapper mapper = ObjectMapper.getDefault();
        try (BufferedReader in = Files.newBufferedReader(Path.of(args[0]), StandardCharsets.UTF_8);
             PrintWriter out = new PrintWriter(Files.newBufferedWriter(Path.of(args[1]), StandardCharsets.UTF_8))) {
            String line;
            while ((line = in.readLine()) != null) {
                if (line.isBlank()) continue;
                @SuppressWarnings("unchecked")
                Map<String, Object> c = mapper.readValue(line, Argument.of(Map.class));
                String schema = (String) c.get("schema"), framing = (String) c.get("framing");
                byte[] input = Base64.getDecoder().decode((String) c.get("input_b64"));
                for (boolean lenient : new boolean[] {false, true}) {
                    Class<?> model = modelOf(schema, lenient);
                    if (model == null || (lenient && !schema.equals("pet"))) continue;
                    Map<String, Object> o = new LinkedHashMap<>();
                    o.put("name", c.get("name"));
                    o.put("schema", schema);
                    o.put("framing", framing);
                    o.put("unknown_enum", lenient ? "null" : "throws");
                    List<Object> recs = new ArrayList<>();
                    if ("array".equals(framing)) {
                        Map<String, Object> r = new LinkedHashMap<>();
                        try {
                            Object v = mapper.readValue(input, Argument.listOf(model));
                            r.put("ok", true);
                            r.put("rewritten_b64", Base64.getEncoder().encodeToString(mapper.writeValueAsBytes(v)));
                        } catch (Throwable t) {
                            r.put("ok", false);
                            r.put("exception", t.getClass().getName());
                            r.put("message", String.valueOf(t.getMessage()));
                        }
                        r.put("whole_document", true);
                        recs.add(r);
                    } else {
                        for (byte[] rec : lines(input)) recs.add(one(mapper, rec, model));
                    }
                    o.put("records", recs);
                    out.println(mapper.writeValueAsString(o));
                }
            }
        }
    }
}
